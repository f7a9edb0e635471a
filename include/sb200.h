/*
 * sb200.h — C ABI of libsarek_b200.so, the B200 (sm_100a) backend for Sarek's
 * dense-GEMM and fused element-wise map path.
 *
 * Every entry point takes plain integers, pointers and sizes so that an OCaml
 * `ctypes-foreign` binding (the style of sarek-cuda/Cuda_bindings.ml:39-87)
 * can bind it with `Foreign.foreign`.  Each function returns an int status:
 * 0 on success, a positive CUDA error code (cudaError_t numbering) when a CUDA
 * call failed, or a negative SB200_ERR_* for errors detected by the library.
 * sb200_last_error_string() describes the last failure on the calling thread.
 *
 * Device pointers are uint64_t (the `device_ptr : nativeint` of
 * spoc/framework/Framework_sig.ml Memory); streams, events and kernels are
 * opaque uint64_t handles; stream 0 is the device's default stream.
 */
#ifndef SB200_H
#define SB200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SB200_API __attribute__((visibility("default")))

/* ---- status codes ----------------------------------------------------- */
#define SB200_OK 0
#define SB200_ERR_INVALID_VALUE (-1)   /* bad argument (null, negative, overflow) */
#define SB200_ERR_INVALID_HANDLE (-2)  /* unknown stream/event/kernel/buffer */
#define SB200_ERR_UNSUPPORTED (-3)     /* IR is not a kernel this backend runs:
                                          the Backend_error.Unsupported_construct
                                          of spoc/framework/Backend_error.ml:21-67 */
#define SB200_ERR_PARSE (-4)           /* malformed IR text */
#define SB200_ERR_ARGS (-5)            /* argument list does not match the kernel */
#define SB200_ERR_BOUNDS (-6)          /* launch would index past a vector's length */
#define SB200_ERR_TIMEOUT (-7)         /* a bounded device-side wait expired */
#define SB200_ERR_NO_DEVICE (-8)       /* no sm_100 device / CUDA unavailable */
#define SB200_ERR_TOO_LARGE (-9)       /* size beyond a stated maximum */
#define SB200_ERR_ALIGNMENT (-10)      /* pointer or leading dimension misaligned */
#define SB200_ERR_COMM (-11)           /* NCCL could not be loaded or one of its calls failed */

/* ---- numeric mode of the GEMM ------------------------------------------ */
#define SB200_MODE_3XTF32 3 /* split accumulation, fp32-grade accuracy (default) */
#define SB200_MODE_TF32 1   /* operands rounded to TF32 once, one MMA per k-step */
#define SB200_MODE_3XF16 4  /* the same three-term split on half-precision panels (fp16 has TF32's 11 significant
                               bits and twice its tensor-core rate): every row of A and every column of B is scaled
                               by a power of two of its own so that its largest magnitude lies in [2^14, 2^15), split
                               hi + lo in fp16, and the accumulators are scaled back exactly.  Same error class as
                               3xTF32 when the elements of a row of A (column of B) lie within about 2^16 of its
                               largest (smaller elements lose low bits of their low part: absolute error below 2^-39
                               of that largest element); about 1.65x as fast at 8192^3.  Every GEMM entry point except
                               sb200_gemm_f32_noalloc takes it. */
#define SB200_MODE_F16 2    /* the high parts of that split alone, one fp16 MMA per k-step: the 11 significant bits of
                               TF32 mode (same error bound) at the fp16 tensor-core rate, with the same per-row and
                               per-column power-of-two scaling; faster than TF32 mode where the tensor work outweighs the conversion pass
                               (from about 4096^3).  Every GEMM entry point except sb200_gemm_f32_noalloc. */
#define SB200_MODE_3XMIXED 5 /* the three-term split of 3xTF32 mode with its two cross terms, hi*lo + lo*hi, on the
                               fp16 pipe: they are 2^-11 of the main term and need 11-bit factors only, which fp16 holds
                               at twice TF32's tensor-core rate.  The main term hi*hi stays a TF32 MMA on the caller's
                               fp32 matrices, so magnitudes are unrestricted where it matters; the fp16 panels of the
                               cross terms carry ONE power-of-two scale per matrix (from its largest magnitude), and
                               the accumulated cross terms are brought back to true units exactly, inside the tensor
                               core (scale-input-d), before the main term is added.  Same error as 3xTF32 for every
                               element within 2^29 of its matrix's largest; an element further down loses bits of its
                               cross terms, in the worst case keeping TF32's 2^-11.  Operands it cannot take (product
                               of the two largest magnitudes above 2^39 or below 2^-58, a NaN or an infinity) are
                               found on the device and computed by the plain 3xTF32 kernels in the same call; small
                               products (below 2^34 multiply-adds, see sb200_set_mixed_min_macs) and operands TMA cannot address use
                               3xTF32 outright.  Every GEMM entry point except sb200_gemm_f32_noalloc takes it. */

/* ---- epilogue activation ------------------------------------------------ */
#define SB200_ACT_NONE 0
#define SB200_ACT_RELU 1 /* if x > 0 then x else 0 */

/* ---- kernel kinds reported by sb200_kernel_kind ----------------------- */
#define SB200_KIND_MAP 1          /* element-wise map (vector_add, triad, fused chains) */
#define SB200_KIND_GEMM_NAIVE 2   /* the matrix_mul IR shape */
#define SB200_KIND_GEMM_TILED 3   /* the matrix_mul_tiled IR shape */
#define SB200_KIND_BLOCK_REDUCE 4 /* shared-memory tree reduction with a fused map (reduce_sum, dot_product) */

/* ---- argument tags for sb200_kernel_launch ---------------------------- */
/* One entry per value the caller's run_source receives, in order: a vector
 * arrives as SB200_ARG_BUFFER followed by SB200_ARG_I32 (its length), scalars
 * as themselves (sarek/sarek/Execute.ml:197-216). */
#define SB200_ARG_BUFFER 0
#define SB200_ARG_I32 1
#define SB200_ARG_I64 2
#define SB200_ARG_F32 3
#define SB200_ARG_F64 4

typedef struct sb200_arg {
  int32_t tag;
  int32_t reserved;
  union {
    uint64_t buffer; /* device pointer */
    int32_t i32;
    int64_t i64;
    float f32;
    double f64;
  } v;
} sb200_arg;

typedef struct sb200_device_info {
  char name[256];
  uint64_t total_mem;
  int32_t cc_major, cc_minor;
  int32_t sm_count;
  int32_t max_threads_per_block;
  int32_t max_shared_per_block; /* opt-in maximum, bytes */
  int32_t warp_size;
  int32_t clock_khz;
  int32_t l2_bytes;
} sb200_device_info;

/* ---- library / device: replaces cuInit, cuDeviceGetCount, cuDeviceGet*,
 *      cuCtxSetCurrent, cuCtxSynchronize (sarek-cuda/Cuda_bindings.ml:90-170,
 *      sarek-cuda/Cuda_api.ml:35-176) ------------------------------------ */
SB200_API int sb200_init(void);
SB200_API int sb200_version(void);
SB200_API const char *sb200_last_error_string(void);
SB200_API int sb200_device_count(int *count);
SB200_API int sb200_device_get_info(int dev, sb200_device_info *out);
SB200_API int sb200_device_set_current(int dev);
SB200_API int sb200_device_synchronize(int dev);

/* ---- memory: replaces cuMemAlloc/cuMemFree/cuMemcpyHtoD/DtoH/DtoD and the
 *      unused async variants (Cuda_bindings.ml:172-258, Cuda_api.ml:191-243).
 *      sb200_mem_free is idempotent (a GC finaliser may free twice,
 *      sarek/core/Gpu_memory.ml:151-178) and waits for the device to go idle. */
SB200_API int sb200_mem_alloc(int dev, uint64_t bytes, uint64_t *dptr);
SB200_API int sb200_mem_free(int dev, uint64_t dptr);
SB200_API int sb200_mem_size(int dev, uint64_t dptr, uint64_t *bytes);
SB200_API int sb200_memset32(int dev, uint64_t dptr, uint32_t value, uint64_t count, uint64_t stream);
/* Synchronous whole-buffer copies, what Transfer.to_device / to_cpu issue (sarek/core/Transfer.ml:229-322).
 * A copy of 16 MiB or more whose host side is pageable memory (a Bigarray) is staged: up to 8 host threads
 * move 4 MiB chunks through pinned slots, each on its own stream, after a device synchronise that keeps the
 * ordering of a default-stream copy.  Measured on B200 (PCIe Gen5 x16): 50 GB/s up, 51 GB/s down, against
 * 11 and 20 GB/s for the plain pageable copy and 55 / 57 GB/s from pinned memory.  SAREK_B200_STAGED_COPY=0
 * switches the staged path off, SAREK_B200_COPY_THREADS sets the thread count (1..8). */
SB200_API int sb200_memcpy_htod(int dev, uint64_t dst, const void *src, uint64_t bytes);
SB200_API int sb200_memcpy_dtoh(int dev, void *dst, uint64_t src, uint64_t bytes);
SB200_API int sb200_memcpy_dtod(int dev, uint64_t dst, uint64_t src, uint64_t bytes);
SB200_API int sb200_memcpy_htod_async(int dev, uint64_t dst, const void *src, uint64_t bytes, uint64_t stream);
SB200_API int sb200_memcpy_dtoh_async(int dev, void *dst, uint64_t src, uint64_t bytes, uint64_t stream);
/* pinned host staging for the transfer path (sarek/core/Transfer.ml:229-322) */
SB200_API int sb200_host_alloc(uint64_t bytes, void **ptr);
SB200_API int sb200_host_free(void *ptr);
/* Pin host memory the caller owns, in place (cudaHostRegister / cudaHostUnregister): later copies from or to it run at
 * the pinned rate (55 GB/s instead of the staged 37-50) and can overlap.  For the owner of a long-lived host array
 * — a Vector over a Bigarray (sarek/core/Vector_storage.ml:18-36), which the plugin registers on its second large
 * transfer and unregisters when the vector is freed.  The range must stay allocated until it is unregistered; both
 * calls are idempotent.  No counterpart in the reference, whose transfers are plain synchronous copies. */
SB200_API int sb200_host_register(void *ptr, uint64_t bytes);
SB200_API int sb200_host_unregister(void *ptr);

/* ---- streams and events: replaces the cuStream and cuEvent families
 *      (Cuda_bindings.ml:260-330, Cuda_api.ml:245-311) ------------------- */
SB200_API int sb200_stream_create(int dev, uint64_t *stream);
SB200_API int sb200_stream_destroy(int dev, uint64_t stream);
SB200_API int sb200_stream_synchronize(int dev, uint64_t stream);
/* adopt a cudaStream_t created elsewhere (e.g. by the host framework) */
SB200_API int sb200_stream_wrap(int dev, uint64_t native_stream, uint64_t *stream);
SB200_API int sb200_event_create(int dev, uint64_t *event);
SB200_API int sb200_event_destroy(int dev, uint64_t event);
SB200_API int sb200_event_record(int dev, uint64_t event, uint64_t stream);
SB200_API int sb200_event_synchronize(int dev, uint64_t event);
SB200_API int sb200_event_elapsed_ms(int dev, uint64_t start, uint64_t stop, float *ms);

/* ---- kernels: replaces generate_source + NVRTC + cuModuleLoadDataEx +
 *      cuLaunchKernel (sarek-cuda/Sarek_ir_cuda.ml:871-929,
 *      sarek-cuda/Cuda_api.ml:315-487, sarek-cuda/Cuda_plugin.ml:174-210).
 *      `ir_text` is the S-expression rendering of a Sarek_ir_types.kernel
 *      (spoc/ir/Sarek_ir_types.ml:230-245).  Compilation recognises the
 *      kernel as a GEMM (naive or tiled shape, with optional fused epilogue)
 *      or an element-wise map; anything else is SB200_ERR_UNSUPPORTED — there
 *      is no fallback path. */
SB200_API int sb200_kernel_compile(int dev, const char *ir_text, const char *name, uint64_t *kernel);
SB200_API int sb200_kernel_destroy(uint64_t kernel);
SB200_API int sb200_kernel_kind(uint64_t kernel, int *kind);
/* human-readable summary of what was recognised (for SAREK_DEBUG=kernel) */
SB200_API int sb200_kernel_describe(uint64_t kernel, char *buf, int buflen);
SB200_API int sb200_kernel_launch(uint64_t kernel, const sb200_arg *args, int nargs,
                                  const uint32_t grid[3], const uint32_t block[3],
                                  uint32_t shared_mem, uint64_t stream);

/* The same launch for arguments that are still in host memory: host_ptrs has one entry per argument; for a
 * SB200_ARG_BUFFER argument a non-null entry means "fill this device buffer from here first" (as many float32 as the
 * length argument that follows it says), every other entry is ignored.  It stands for the reference's
 * Transfer.to_device of each argument followed by the launch (sarek/sarek/Execute.ml:520-543,
 * sarek/core/Transfer.ml:229-268) in one call, which lets the library overlap the two: when the kernel is a recognised
 * matmul whose launch covers the whole product and the host arrays are pinned or registered, B and the bias go first and
 * A and C follow in row blocks, each block's GEMM starting when its rows have arrived; the ahead-of-time element-wise
 * operators on vectors of 16 MiB or more go chunk by chunk the same way; otherwise the vectors are copied whole (staged
 * when pageable and large) and the kernel is launched behind them.  The call returns when every
 * upload has completed, so the host arrays may be changed at once; the kernel may still be running on `stream`. */
SB200_API int sb200_kernel_launch_from_host(uint64_t kernel, const sb200_arg *args, int nargs,
                                            const void *const *host_ptrs, void *const *host_out,
                                            int32_t *prefetched, const uint32_t grid[3],
                                            const uint32_t block[3], uint32_t shared_mem, uint64_t stream);
/* host_out and prefetched (both null, or both tables of nargs entries) extend the call to the way back: a non-null
 * host_out entry of a buffer argument names the host array the caller keeps that vector's host copy in.  The reference
 * marks every vector argument stale on the host after a launch (sarek/sarek/Execute.ml:546-553) and downloads it when
 * the host next reads it (sarek/core/Transfer.ml:272-322); a stale host copy may therefore be overwritten early.  For
 * the vector a recognised matmul writes (or the outputs of an element-wise operator that runs by chunks), when that
 * array is pinned or registered, the library sends the result back behind the kernel (block by block on the
 * pipelined routes) and sets prefetched[i] = 1; every other entry is
 * set to 0 and the caller downloads as before.  The host copy is complete once sb200_prefetch_wait has returned. */
SB200_API int sb200_prefetch_wait(int dev);

/* ---- IR fusion: the host-side rewrite of sarek/sarek/Sarek_fusion.ml
 *      (can_fuse :401-431, fuse :459-547, fuse_pipeline :570-598) on IR text.
 *      Results are written to `out` (NUL-terminated, at most outlen bytes). */
SB200_API int sb200_ir_can_fuse(const char *producer, const char *consumer, const char *intermediate, int *result);
SB200_API int sb200_ir_fuse(const char *producer, const char *consumer, const char *intermediate, char *out, int outlen);
SB200_API int sb200_ir_fuse_pipeline(const char *const *kernels, int count, char *out, int outlen, char *eliminated, int elimlen);
/* should_fuse (Sarek_fusion.ml:1068-1098): decision is "Fuse", "DontFuse" or "MaybeFuse" */
SB200_API int sb200_ir_should_fuse(const char *producer, const char *consumer, const char *intermediate,
                                   char *decision, int declen, char *reason, int reasonlen);
/* auto_fuse_pipeline (Sarek_fusion.ml:1133-1165): eliminated arrays comma-separated, skipped reasons one per line */
SB200_API int sb200_ir_auto_fuse_pipeline(const char *const *kernels, int count, char *out, int outlen,
                                          char *eliminated, int elimlen, char *skipped, int skiplen);
/* analyze (Sarek_fusion.ml:340-354): one line per array "read|write NAME one_to_one|stencil[..]|gather|unknown",
 * then "barriers yes|no" */
SB200_API int sb200_ir_analyze(const char *kernel, char *out, int outlen);
/* The other fusion forms of the reference, selected by `kind`:
 *   SB200_FUSE_PLAIN      can_fuse / fuse                          (Sarek_fusion.ml:401-547)
 *   SB200_FUSE_REDUCTION  can_fuse_reduction / fuse_reduction       (:636-757)
 *   SB200_FUSE_STENCIL    can_fuse_stencil / fuse_stencil           (:795-1018)
 *   SB200_FUSE_TRY        try_fuse: reduction, else plain           (:759-766)
 *   SB200_FUSE_TRY_ALL    try_fuse_all: reduction, stencil, plain   (:1022-1030)
 *   SB200_FUSE_GUARDED    no counterpart in the reference: fuses kernels of the form its own benchmarks use,
 *                         `let tid = global_thread_id in if tid < n then out.(tid) <- e`, which the reference's
 *                         pass leaves unfused (find_write_expr stops at a conditional, :370-375; the two kernels'
 *                         `tid` have different ids, :38).  Index lets are inlined and the guards peeled; the
 *                         producer must be unguarded or guarded exactly as the consumer (parameters compared by
 *                         name), the consumer must read the intermediate only at the producer's store index.
 *                         Replaced reads of a float32 intermediate are wrapped in (intrinsic (B200) stored_f32 e), "e as
 *                         the vector would have held it", so the fused kernel rounds where the unfused pair stored.
 * For the TRY and GUARDED kinds *fused is 0 when nothing was fused (out is then empty); for GUARDED
 * sb200_last_error_string then says which condition failed. */
#define SB200_FUSE_PLAIN 0
#define SB200_FUSE_REDUCTION 1
#define SB200_FUSE_STENCIL 2
#define SB200_FUSE_TRY 3
#define SB200_FUSE_TRY_ALL 4
#define SB200_FUSE_GUARDED 5
SB200_API int sb200_ir_can_fuse_as(const char *producer, const char *consumer, const char *intermediate, int kind, int *result);
SB200_API int sb200_ir_fuse_as(const char *producer, const char *consumer, const char *intermediate, int kind,
                               char *out, int outlen, int *fused);
/* fuse_pipeline (Sarek_fusion.ml:570-598: greedy, left to right, first candidate array) with the fusion form of
 * each step chosen by `kind`; with SB200_FUSE_GUARDED a chain of benchmark-form kernels collapses into one kernel. */
SB200_API int sb200_ir_fuse_pipeline_as(const char *const *kernels, int count, int kind, char *out, int outlen,
                                        char *eliminated, int elimlen);

/* ---- direct operators (what a recognised kernel launch dispatches to) ---
 * D[M x N] = act(alpha * A[M x K] . B[K x N] + beta * C[M x N] + bias[N]),
 * all row-major float32 with leading dimensions in elements; C and bias may
 * be 0.  D may alias C.  Replaces the matrix_mul / matrix_mul_tiled kernels
 * (benchmarks/bench_matrix_mul.ml:55-73, bench_matrix_mul_tiled.ml:55-94).
 * Operands that lie inside buffers from sb200_mem_alloc are checked against the end of their buffer
 * (SB200_ERR_BOUNDS, nothing is launched); memory from other allocators is taken at the caller's word.
 * Calls may be issued on any streams of the device: those that use the library's scratch (3xTF32 mode, or operands
 * TMA cannot address as they lie) are ordered against each other across streams by the library, the others run
 * concurrently.
 * Once a first call with the same sizes has sized the library's scratch, a call enqueues nothing but kernel launches
 * (the GEMM launch carries the programmatic-stream-serialization attribute), so it can be captured into a CUDA graph
 * together with the map operators and replayed (tests/test_gpu_gemm.py). */
SB200_API int sb200_gemm_f32(int dev, uint64_t stream, int mode,
                             int64_t M, int64_t N, int64_t K,
                             uint64_t A, int64_t lda, uint64_t B, int64_t ldb,
                             uint64_t D, int64_t ldd,
                             float alpha, uint64_t C, int64_t ldc, float beta,
                             uint64_t bias, int act);
/* Same operator and arguments as sb200_gemm_f32, for callers that must not
 * allocate device memory: a host framework whose caching allocator already owns
 * all of the GPU's memory (any further cudaMalloc fails), or a caller that
 * cannot take the device-wide synchronisation of cudaMalloc/cudaFree while its
 * other streams are busy.  This entry point has no counterpart in the
 * reference.  It allocates nothing: the TF32 operand panels live in a fixed
 * 32 MiB device array inside the library image (held by every GPU that loads
 * the library, until exit).  Sizes whose panels do not fit, (M+N)*roundup(K,32)*4
 * bytes (x2 in 3xTF32 mode), return SB200_ERR_TOO_LARGE.  All calls on a device
 * share the array and it keeps the last call's contents (each call rewrites
 * all it reads); calls that overlap on the GPU race on it.  The first call on a
 * device looks up the array's address and should come before any stream
 * capture.  Every call waits on `stream` until its kernels have finished and reads
 * a status word back with a synchronous copy: do not issue it on a stream that is
 * being captured.  Operand extents are checked as in sb200_gemm_f32. */
SB200_API int sb200_gemm_f32_noalloc(int dev, uint64_t stream, int mode,
                                     int64_t M, int64_t N, int64_t K,
                                     uint64_t A, int64_t lda, uint64_t B, int64_t ldb,
                                     uint64_t D, int64_t ldd,
                                     float alpha, uint64_t C, int64_t ldc, float beta,
                                     uint64_t bias, int act);
/* Row-sharded product with the gather fused into the store.  Each GPU computes the M_local rows of D that start
 * at global row `row_offset` and writes every element to the same position of `n_copies` (1..8) full-size copies
 * of D, whose base addresses are d_copies[]: entry 0 this GPU's own copy, the others the peers' copies mapped
 * into this process (sb200_ipc_open) — plain stores over NVLink from the epilogue, so the all-gather of the
 * row blocks overlaps the tensor-core work instead of following it.  When every GPU has returned from its
 * stream synchronise and the ranks have met at a host barrier, each copy holds the whole D.  The reference has
 * no multi-GPU path (sarek/core/Vector.ml:284-296 leaves gather a stub); this is the gathered-result form of
 * the row-block sharding described for it.  A, C (M_local rows) and B, bias (whole) are local. */
SB200_API int sb200_gemm_f32_gather(int dev, uint64_t stream, int mode, int64_t M_local, int64_t N, int64_t K,
                                    uint64_t A, int64_t lda, uint64_t B, int64_t ldb,
                                    const uint64_t *d_copies, int n_copies, int64_t row_offset, int64_t ldd,
                                    float alpha, uint64_t C, int64_t ldc, float beta, uint64_t bias, int act);
/* Sharing a buffer obtained from sb200_mem_alloc with the other processes of the node (one process per GPU):
 * export writes a 64-byte handle to pass to the peers by any host channel; open maps the peer's buffer into
 * this process (peer access over NVLink is enabled on first use) and returns a device pointer usable in
 * d_copies[]; close unmaps it.  Thin wrappers of cudaIpcGetMemHandle / OpenMemHandle / CloseMemHandle. */
SB200_API int sb200_ipc_export(int dev, uint64_t dptr, void *handle64);
SB200_API int sb200_ipc_open(int dev, const void *handle64, uint64_t *dptr);
SB200_API int sb200_ipc_close(int dev, uint64_t dptr);

/* ---- one process, several GPUs ------------------------------------------------------------------------
 * The reference's host is a single process whose multi-device model is to partition a vector and launch once
 * per device (sarek/core/Vector.ml:273-296, split rule sarek/core/Vector_storage.ml:261-272: the first
 * `total mod parts` parts get one element more); it binds peer access (sarek-cuda/Cuda_bindings.ml:472-493)
 * and never uses it.  A group is that model for the GEMM path: 1 to 8 distinct GPUs of this process (devices ==
 * NULL means 0..ngpus-1), each with its own streams; with more than one GPU the library loads NCCL (a copy the
 * process has already loaded, else the file SAREK_B200_NCCL names, else libnccl.so.2 from the library path)
 * and creates one communicator per GPU (ncclCommInitAll), and enables peer access between the
 * members.  Errors in the arguments (size, device index out of range or repeated) are reported before any GPU
 * work; SB200_ERR_COMM means NCCL could not be loaded or failed. */
SB200_API int sb200_group_create(int ngpus, const int *devices, uint64_t *group);
SB200_API int sb200_group_destroy(uint64_t group);
SB200_API int sb200_group_size(uint64_t group, int *ngpus);
SB200_API int sb200_group_device(uint64_t group, int index, int *dev);
/* rows [first, first+count) of part `index` when `total` rows are split into `parts` (Vector_storage.ml:261-272) */
SB200_API int sb200_row_block(int64_t total, int parts, int index, int64_t *first, int64_t *count);
/* Row-sharded D = act(alpha*A.B + beta*C + bias) on device-resident operands.  a_shards[i] / c_shards[i] (table or
 * entries may be 0 when there is no C) hold member i's row block of A / C on member i's GPU; B (ldb == N when the
 * group has more than one GPU) and bias lie on the first member's GPU and are replicated into group-owned buffers
 * on the others with ncclBroadcast at every call, unless SB200_SHARD_B_RESIDENT says that the replicas made by the
 * previous call (same B, bias and sizes) are still valid.  Without a gather flag d[i] is member i's row block of D.
 * With SB200_SHARD_GATHER_FUSED or SB200_SHARD_GATHER_NCCL d[i] is a whole M x N copy of D on member i's GPU and
 * every copy is complete on return: FUSED stores each finished tile into all copies from the GEMM epilogue (plain
 * peer stores over NVLink, overlapping the tensor-core work; needs peer access between all members), NCCL runs
 * the GEMM into the member's own rows and then gathers in place (ncclAllGather, or one ncclBroadcast per block
 * when M does not divide; needs ldd == N).  All forms give the same bits.  The call returns when every member's
 * stream has finished; sb200_group_last_ms then gives the device time of the call (CUDA events around the
 * member's work, maximum over members). */
#define SB200_SHARD_GATHER_FUSED 1
#define SB200_SHARD_GATHER_NCCL 2
#define SB200_SHARD_B_RESIDENT 4
SB200_API int sb200_gemm_sharded(uint64_t group, int mode, int64_t M, int64_t N, int64_t K,
                                 const uint64_t *a_shards, int64_t lda, uint64_t b, int64_t ldb,
                                 const uint64_t *d, int64_t ldd, float alpha,
                                 const uint64_t *c_shards, int64_t ldc, float beta, uint64_t bias, int act, int flags);
SB200_API int sb200_group_last_ms(uint64_t group, float *ms);
/* The same on HOST operands, the multi-GPU form of sb200_gemm_f32_host below: B crosses PCIe once, a band of
 * rows over each GPU's link, and is assembled on every GPU over NVLink (ncclAllGather in place; the bias goes to the
 * first GPU and is broadcast); each GPU pulls only its own rows of A and C
 * and pushes only its own rows of D over its own PCIe link, driven by a host thread of its own, in row chunks so
 * that copies in, GEMM and copies out overlap.  Pinned memory is copied asynchronously, contiguous pageable
 * memory through the staged copier.  Returns when D is complete in host memory.  Replaces, for several devices,
 * Transfer.to_device of every argument, one launch per device and Transfer.to_cpu
 * (sarek/core/Transfer.ml:229-322, sarek/core/Vector.ml:273-296). */
SB200_API int sb200_gemm_sharded_host(uint64_t group, int mode, int64_t M, int64_t N, int64_t K,
                                      const float *A, int64_t lda, const float *B, int64_t ldb,
                                      float *D, int64_t ldd, float alpha, const float *C, int64_t ldc,
                                      float beta, const float *bias, int act);

/* The same operator on HOST operands.  Pinned memory (sb200_host_alloc) gives full
 * overlap with asynchronous copies: 15.9 ms at 8192^3.  Contiguous pageable operands
 * (a Bigarray) are moved block by block by the staged copier — host threads through
 * pinned slots, copy-out on a thread of its own — beside the GEMM of the block
 * before: 27.0 ms at 8192^3, against 93.6 ms with plain pageable copies; strided
 * pageable operands take the plain copies.  Replaces the reference's sequence
 * Transfer.to_device of every argument, launch, Transfer.to_cpu of the result
 * (sarek/core/Transfer.ml:229-322, sarek/sarek/Execute.ml:520-543) with one call
 * in which host-to-device copies, the GEMM of the row blocks that have arrived
 * and device-to-host copies of finished blocks overlap.  Returns when D is
 * complete in host memory. */
SB200_API int sb200_gemm_f32_host(int dev, int mode, int64_t M, int64_t N, int64_t K,
                                  const float *A, int64_t lda, const float *B, int64_t ldb,
                                  float *D, int64_t ldd, float alpha, const float *C, int64_t ldc,
                                  float beta, const float *bias, int act);
/* bytes of library-owned scratch sb200_gemm_f32 needs for these sizes */
SB200_API int sb200_gemm_workspace_bytes(int mode, int64_t M, int64_t N, int64_t K, uint64_t *bytes);
/* how sb200_gemm_f32 would run these sizes on a device with sm_count SMs, as text:
 * "pair|single direct|panels tile=RxC stages=S tiles=T waves=W workspace=BYTES launches=L".
 * addressable = operands 16-byte aligned with row strides that are multiples of 4 floats.  Needs no GPU. */
SB200_API int sb200_gemm_describe(int mode, int64_t M, int64_t N, int64_t K, int addressable, int sm_count,
                                  char *out, int outlen);

/* c = a + b  (benchmarks/bench_vector_add.ml:47-55) */
SB200_API int sb200_vector_add_f32(int dev, uint64_t stream, uint64_t c, uint64_t a, uint64_t b, int64_t n);
/* a = b + c * scalar  (benchmarks/bench_stream_triad.ml:22-31) */
SB200_API int sb200_stream_triad_f32(int dev, uint64_t stream, uint64_t a, uint64_t b, uint64_t c, float scalar, int64_t n);
/* fused chain a = b + scalar*c ; d = a*a + b in one pass; a_out may be 0 when
 * the intermediate is eliminated (sarek/sarek/Sarek_fusion.ml:490-499). */
SB200_API int sb200_chain_triad_square_f32(int dev, uint64_t stream, uint64_t d, uint64_t a_out, uint64_t b, uint64_t c, float scalar, int64_t n);

/* default numeric mode for GEMM kernels launched through sb200_kernel_launch
 * (also read once from the environment variable SAREK_B200_MODE=3xtf32|tf32|3xf16|f16) */
SB200_API int sb200_set_mode(int mode);
SB200_API int sb200_get_mode(int *mode);
/* which tensor-core kernel sb200_gemm_f32 launches: 0 = automatic (CTA pairs on
 * 256-row tiles when M > 128 or when the operands are 16-byte aligned with row
 * strides that are multiples of 4 floats, so that the kernel reads them directly;
 * else single-CTA 128x256 tiles fed from prepared panels), 1 = always
 * single-CTA tiles, 2 = always CTA pairs, 3 = CTA pairs fed from prepared
 * operand panels even where TF32 mode could read the caller's matrices
 * directly.  Also SAREK_B200_GEMM=single|pair|pair-panels.  All variants round
 * operands to TF32 the same way (nearest-even) and sum k ascending, so their
 * results agree to the last bit. */
SB200_API int sb200_set_gemm_variant(int variant);
/* tile columns of the CTA-pair kernel: 0 = automatic (256, or 128 / 64 for problems with too few 256-column
 * tiles to occupy the SMs), else 64, 128 or 256.  Also SAREK_B200_TILE_N.  Results do not depend on it. */
SB200_API int sb200_set_gemm_tile_n(int tile_n);
/* The soft lockstep of the CTA-pair kernel: every 64 stages of the k-loop each pair counts itself into an epoch counter
 * in global memory and waits, 4 us at most and then regardless, for the other pairs of the launch, so that the pairs of a
 * wave, which share rows of A and columns of B through L2, stay within L2's reach of one another (DRAM reads of the
 * 8192^3 launch 4.8 GB instead of 6.6 GB; 35 instead of 131 GB at K = 32768).  A hint: results do not depend on it.
 * -1 = on for k-loops of 128 stages or more except in TF32 mode, whose short stages make the waits weigh more than the
 * traffic they save (default), 0 = off, 1 = always.  Also SAREK_B200_LOCKSTEP=0|1. */
SB200_API int sb200_set_lockstep(int setting);
/* SB200_MODE_3XMIXED hands products of fewer than this many multiply-adds (M*N*K) to 3xTF32, whose two launches cost
 * less than the mixed mode's seven on small problems; 0 restores the default (2^34).  A tuning and test knob. */
SB200_API int sb200_set_mixed_min_macs(int64_t macs);
/* The plan SB200_MODE_3XMIXED makes on the device from the largest magnitudes of A and B (no GPU needed): out[0] = 1
 * when the mixed kernel takes the operands (0: the 3xTF32 kernels behind it do), out[1] = rescale stages, out[2] = the
 * first main-term MMA's scale, out[3], out[4] = the binary exponents the fp16 panels of A and B are scaled by. */
SB200_API int sb200_mixed_plan(float max_a, float max_b, int32_t out[5]);

/* L2 eviction policies the GEMM kernels attach to their memory instructions (a per-instruction cache hint;
 * no device setting is touched): three 2-bit fields, each 0 = normal, 1 = evict first, 2 = evict last —
 * bits 0-1 the TMA loads of A (high and low parts), bits 2-3 the TMA loads of B, bits 4-5 the epilogue's reads
 * of C and writes of D.  -1 returns to the built-in default (also SAREK_B200_L2_POLICY).  Results do not
 * depend on it.  No counterpart in the reference, whose generated kernels carry no cache hints. */
SB200_API int sb200_set_l2_policy(int bits);

/* seeded synthetic data written on the device: kind 0 U[-1,1), 1 U[-0.1,0.1),
 * 2 N(0,sigma); element i of the stream is a pure function of (seed, stream_id,
 * first + i). */
SB200_API int sb200_fill_f32(int dev, uint64_t stream, uint64_t dptr, int64_t n,
                             uint64_t seed, uint64_t stream_id, int kind, double sigma, int64_t first);

/* kernel profiling: the enable_profiling / disable_profiling members of
 * Framework_sig.BACKEND (spoc/framework/Framework_sig.ml:280-282;
 * sarek-cuda/Cuda_plugin_base.ml:294-300).  While enabled, every GEMM call
 * records CUDA events on its launch stream around the operand-preparation
 * kernels and around the tensor-core kernel; sb200_profile_gemm_read waits for
 * the recorded calls, returns their count and summed durations and clears the
 * record. */
SB200_API int sb200_enable_profiling(int on);
SB200_API int sb200_profile_gemm_read(int dev, uint64_t *calls, double *prep_ms, double *main_ms);

/* Failure-detection self-test, fault-free: launches one block whose only thread waits, for at most
 * limit_ms (1..1000), on a barrier that nothing signals, then gives up the way the GEMM pipeline's roles
 * do.  The next sb200_device_synchronize / sb200_stream_synchronize / sb200_memcpy_dtoh on that device
 * returns SB200_ERR_TIMEOUT once, and the device stays usable.  No counterpart in the reference, whose
 * calls are synchronous and carry no device-side waits. */
SB200_API int sb200_selftest_wait_timeout(int dev, uint32_t limit_ms);

/* number of kernels this library has launched on this thread's behalf since
 * load (monotonic; used by benchmarks to report launch counts) */
SB200_API int sb200_launch_count(uint64_t *count);

#ifdef __cplusplus
}
#endif
#endif /* SB200_H */
