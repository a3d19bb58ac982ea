/* C ABI of the Basalt sm_100a device path: the Backend boundary (BIR text in, PTX text out) and
 * the launch runtime (CUDA Driver API, JIT load, streams, sharding, NCCL).
 *
 * Every entry point states the reference interface it stands in for (paths inside the reference
 * project).  All functions are re-entrant unless noted; none keeps a pointer passed to it beyond
 * the call.  Return value: 0 on success unless documented otherwise.
 */
#ifndef BASALT_B200_H
#define BASALT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

/* ------------------------------------------------------------------------------------------
 * Backend: the `Backend` trait (crates/basalt-backend/src/backend.rs:144-157) as implemented by
 * `Ptx` (crates/basalt-ptx/src/emit.rs:1973-1994).  `&Module` crosses as BIR text, the form the
 * reference CLI itself accepts (crates/basalt-cli/src/main.rs:517-520).
 * ---------------------------------------------------------------------------------------- */

/* EmitOpts (backend.rs:123-137). target_variant: NULL or "sm_100a". opt_level: 0 lowers one to
 * one like the reference, 1/2 run the vectorising passes (2 is the default when opts is NULL).
 * out_name_hint and snap are accepted and ignored, as Ptx::emit ignores them (emit.rs:1988). */
typedef struct basalt_emit_opts {
    const char *target_variant;
    int opt_level;
    const char *out_name_hint;
    int snap;
} basalt_emit_opts;

/* Diag (crates/basalt-diag/src/diag.rs:62-66): the stable E-code string (ecode.rs:148-181) and
 * the argument the reference would render into the message template. */
typedef struct basalt_diag {
    char code[8];
    char message[504];
} basalt_diag;

/* Backend::name (backend.rs:146). */
const char *basalt_b200_name(void);

/* Backend::supports (backend.rs:148-151; Ptx: emit.rs:1981-1986). Returns 1 when the module can
 * be emitted, 0 when refused (ecode_out receives e.g. "E090"), -1 when the text is not BIR
 * (ecode_out receives "E400", crates/basalt-cli/src/main.rs:308-309). */
int basalt_b200_supports(const char *bir, size_t len, char ecode_out[8]);

/* Backend::emit (backend.rs:152-156; Ptx: emit.rs:1988-1993). On success *ptx_out is a
 * NUL-terminated, malloc'd PTX module (free with basalt_b200_free) and the result is 0; on
 * refusal the result is 1 and diag_out is filled. Deterministic for a given (bir, opts). */
int basalt_b200_emit(const char *bir, size_t len, const basalt_emit_opts *opts, char **ptx_out,
                     size_t *ptx_len, basalt_diag *diag_out);

/* The module as the emitter lowers it, after inlining and the vectorising passes, printed as BIR.
 * No reference counterpart (the reference has no backend passes); exists so the passes can be
 * checked against the CPU oracle. */
int basalt_b200_optimize(const char *bir, size_t len, const basalt_emit_opts *opts, char **bir_out,
                         size_t *bir_len, basalt_diag *diag_out);

/* basalt_bir::parse followed by basalt_bir::print (crates/basalt-bir/src/lib.rs:79-85): the
 * round-trip the reference tests in crates/basalt-bir/tests/roundtrip.rs. */
int basalt_b200_roundtrip(const char *bir, size_t len, char **bir_out, size_t *bir_len,
                          basalt_diag *diag_out);

/* The front half of the reference CLI's CUDA-C lane (crates/basalt-cli/src/main.rs:286-327:
 * preprocess, parse, type-check, lower to BIR) for the subset of the language device kernels are
 * written in: crates/basalt-frontend-c plus crates/basalt-sema/src/{checker,lower}.rs.  On success
 * *bir_out is the slot-form BIR text of the translation unit (the form sema hands to the passes,
 * lower.rs:882-898, 992-1063), ready for basalt_b200_emit.  A refusal carries the reference's
 * front-end codes: E200/E201/E202 lexical and syntax, E300-E304 and E308 semantic. */
int basalt_b200_compile_cuda(const char *src, size_t len, char **bir_out, size_t *bir_len,
                             basalt_diag *diag_out);

/* The front half of the reference CLI's Triton lane (crates/basalt-cli/src/main.rs:329-372:
 * parse, check_triton, lower_triton) for `@triton.jit` kernels, re-thought for a GPU: a program
 * is a CTA, elementwise tile code is a loop over lanes strided by the CTA's thread count, and
 * tl.dot is BIR's `mma` (the reference lowers it to a scalar triple loop because its back ends
 * refuse `mma`, crates/basalt-sema/src/triton_lower.rs:9-31).  `bindings` is NULL or a
 * space-separated list: `NAME=<int>` gives a tl.constexpr parameter without a literal default its
 * compile-time value, `NAME=*f16|*f32|*f64|*i64` the element type behind a pointer parameter
 * (f32 when absent, the reference's assumption, triton_lower.rs:72-84), `num_warps=<n>` the CTA
 * size the kernel is compiled for (Triton's launch option).  The kernel ABI is the reference's
 * (triton_lower.rs:517-551): parameters in source order, pointers as ptr.global, scalars as i64,
 * constexpr parameters with a literal default dropped.  Refusals: E200/E201/E202, E300-E307. */
int basalt_b200_compile_triton(const char *src, size_t len, const char *bindings, char **bir_out,
                               size_t *bir_len, basalt_diag *diag_out);

void basalt_b200_free(void *p);

/* ------------------------------------------------------------------------------------------
 * Runtime: crates/basalt-runtime/src/{driver,context,module,ffi,error}.rs.
 * ---------------------------------------------------------------------------------------- */
typedef struct basalt_rt_driver basalt_rt_driver;     /* CudaDriver   (driver.rs:94-163)   */
typedef struct basalt_rt_ctx basalt_rt_ctx;           /* CudaContext  (context.rs:30-91)   */
typedef struct basalt_rt_module basalt_rt_module;     /* CudaModule   (module.rs:11-60)    */
typedef struct basalt_rt_function basalt_rt_function; /* CudaFunction (module.rs:62-123)   */
typedef struct basalt_rt_buffer basalt_rt_buffer;     /* DeviceBuffer (context.rs:95-168)  */
typedef struct basalt_rt_comm basalt_rt_comm;         /* no counterpart: the reference is single-GPU */

/* CudaError (error.rs:9-22). kind: 1 DriverNotFound, 2 SymbolNotFound, 3 DriverCallFailed,
 * 4 a host-side check of this runtime (bounds, arguments), 5 NCCL. */
typedef struct basalt_rt_error {
    int kind;
    int code;           /* CUresult / ncclResult_t */
    char call[64];      /* e.g. "cuModuleLoadData" */
    char message[440];
} basalt_rt_error;
/* The error of the calling thread's most recent failed runtime call. */
void basalt_rt_last_error(basalt_rt_error *out);

/* CudaDriver::load (driver.rs:104-133): dlopen libcuda.so.1 / libcuda.so, resolve entry points
 * with their _v2 fallbacks, cuInit(0). */
int basalt_rt_driver_load(basalt_rt_driver **out);
void basalt_rt_driver_unload(basalt_rt_driver *drv);
/* CudaDriver::device_count (driver.rs:136-141). */
int basalt_rt_device_count(basalt_rt_driver *drv, int *count);
/* CudaDriver::create_context (driver.rs:143-159). Retains the device's primary context instead
 * of creating a new one, so memory and streams are shared with any CUDA runtime user (PyTorch,
 * NCCL) in the process. */
int basalt_rt_ctx_create(basalt_rt_driver *drv, int device_index, basalt_rt_ctx **out);
void basalt_rt_ctx_destroy(basalt_rt_ctx *ctx);
/* cuDeviceGetAttribute; attr is a CUdevice_attribute value. */
int basalt_rt_device_attr(basalt_rt_ctx *ctx, int attr, int *value);

/* CudaContext::load_module (context.rs:43-61): cuModuleLoadDataEx on the PTX text; the driver's
 * JIT runs here. The JIT's error log is kept for basalt_rt_last_error. Also reads the
 * `//!basalt.plan` lines the emitter writes for kernels that need tensor maps. */
int basalt_rt_module_load(basalt_rt_ctx *ctx, const char *ptx, basalt_rt_module **out);
void basalt_rt_module_unload(basalt_rt_module *mod);
/* CudaModule::get_function (module.rs:22-44). */
int basalt_rt_get_function(basalt_rt_module *mod, const char *name, basalt_rt_function **out);

/* CudaContext::alloc (context.rs:64-76). */
int basalt_rt_alloc(basalt_rt_ctx *ctx, size_t bytes, basalt_rt_buffer **out);
void basalt_rt_buffer_free(basalt_rt_buffer *buf);
/* DeviceBuffer::device_ptr / len (context.rs:142-150). */
uint64_t basalt_rt_buffer_ptr(const basalt_rt_buffer *buf);
size_t basalt_rt_buffer_size(const basalt_rt_buffer *buf);
/* DeviceBuffer::copy_from_host / copy_to_host (context.rs:104-140): refuse (kind 4) when bytes
 * exceeds the buffer. stream NULL = synchronous copy like the reference; otherwise asynchronous
 * on that CUstream. */
int basalt_rt_copy_from_host(basalt_rt_buffer *buf, const void *host, size_t bytes, void *stream);
int basalt_rt_copy_to_host(const basalt_rt_buffer *buf, void *host, size_t bytes, void *stream);
/* Page-locked host memory for asynchronous copies (no counterpart; the reference copies from
 * pageable memory). */
int basalt_rt_host_alloc(basalt_rt_ctx *ctx, size_t bytes, void **out);
void basalt_rt_host_free(basalt_rt_ctx *ctx, void *p);

/* CudaFunction::launch (module.rs:77-122): cuLaunchKernel with params[i] pointing at the i-th
 * kernel parameter, in the BIR parameter order. Unlike the reference it takes a stream and does
 * not synchronise; pass stream NULL and call basalt_rt_ctx_sync for the reference behaviour.
 * For a kernel with a launch plan, the tensor-map parameters are built from the pointer and size
 * parameters and appended here; the caller still passes only the BIR parameters.
 * Launches of the FFMA matmul that work a sparse last wave off with stream units (partial sums
 * along K) share one workspace per context (two 64 KB tiles per unit; a launch that needs more than
 * an earlier one did gets a new allocation, and the outgrown one lives until the context is destroyed,
 * so that earlier launches and captured graphs stay valid); the runtime orders them itself (each such launch waits, on its own stream, for the
 * previous one wherever that ran), so callers may issue them from any streams and host threads. */
int basalt_rt_launch(basalt_rt_function *fn, const uint32_t grid[3], const uint32_t block[3],
                     uint32_t shared_mem_bytes, void *stream, void **params);
/* basalt_rt_launch for one rank of a row-sharded matmul whose result every rank wants whole: compute
 * and gather in ONE kernel.  peer_out[i] (0 <= n_peers <= 7) is the value the kernel's output pointer
 * parameter has on another rank, as an address valid on this device (basalt_rt_ipc_open); the
 * kernel stores every tile of its result at its own output pointer and, at the same offset, behind
 * each peer address over NVLink (plain line-sized stores from the SMs while the next tiles are being
 * computed -- in the tcgen05 matmul by two relay warps per CTA that read each finished tile back from
 * L2, so that the epilogue never waits on a link; no copy engine, no library collective), and ends
 * with a system-scope fence.  A stream-ordered basalt_rt_peer_allreduce_max_i32 afterwards is the barrier after which
 * every rank holds every rank's rows.  The peers are served in the order given: pass rank + 1,
 * rank + 2, ... (mod the group size), so that at every moment no two ranks store into the same
 * receiver.  Only kernels the emitter lowered with a gathering epilogue
 * take it (the fp32 FFMA matmul; the fp16 tcgen05 matmul through its two-SM entry, so the grid must
 * be even in x and y); any other kernel is refused (kind 4).  No counterpart in the reference, which
 * has no multi-GPU path (crates/basalt-runtime/src/ffi.rs:38-42). */
int basalt_rt_launch_gather(basalt_rt_function *fn, const uint32_t grid[3], const uint32_t block[3],
                            uint32_t shared_mem_bytes, void *stream, void **params, const uint64_t *peer_out,
                            int n_peers);
/* basalt_rt_launch_gather through an NVLink multicast mapping (NVLS): multicast_out is the value the kernel's output
 * pointer parameter would have inside a multicast mapping that covers the same result buffer on every GPU of the group,
 * this one included (cuMulticastCreate / cuMulticastBindMem over buffers of one size; 16-byte aligned; the caller
 * builds the mapping, e.g. torch.distributed._symmetric_memory's multicast_ptr).  The kernel still writes this GPU's
 * result with plain stores and sends each finished tile once, with multimem.st, to be replicated by the switch: one
 * copy leaves the GPU instead of one per peer.  Completion is the caller's barrier, as for basalt_rt_launch_gather.
 * A rank must not exit while its memory is bound to a multicast object that other ranks still use.  No counterpart
 * in the reference. */
int basalt_rt_launch_gather_multicast(basalt_rt_function *fn, const uint32_t grid[3], const uint32_t block[3],
                                      uint32_t shared_mem_bytes, void *stream, void **params, uint64_t multicast_out);
/* Grid and block the emitter planned for this kernel (0 when the kernel has no plan and the
 * caller chooses, as with the reference). */
int basalt_rt_planned_geometry(basalt_rt_function *fn, void **params, uint32_t grid[3], uint32_t block[3],
                               uint32_t *shared_mem_bytes);
/* Resident CTAs per SM for this kernel at the given block size (cuOccupancyMaxActiveBlocksPer-
 * Multiprocessor) and the device's SM count: a grid of their product is exactly one wave. No
 * counterpart in the reference, which leaves grid sizing to its tests. */
int basalt_rt_occupancy(basalt_rt_function *fn, uint32_t block_threads, uint32_t shared_mem_bytes, int *ctas_per_sm,
                        int *sm_count);
/* The schedule basalt_rt_launch gives an FFMA matmul whose plan says `tail=` (kernels/sgemm.cu describes the scheme):
 * out = {full, per, units}.  Of `tiles` 128x128 tiles on `slots` resident CTAs, tiles [0, full) run whole, one CTA each;
 * the rest are worked off by `units` stream units of `per` K slabs (16 columns of A) each, the tail tiles' slabs laid end
 * to end, in `rounds` rounds of one unit per slot.  per = units = 0 and full = tiles when nothing would be gained.  A pure
 * function (no context, no device): exported so that the index arithmetic of the units can be checked without a GPU.
 * No counterpart in the reference. */
void basalt_rt_tail_plan(uint32_t tiles, uint32_t slots, uint32_t k_extent, uint32_t rounds, uint32_t out[3]);
/* Switches one of the runtime's launch policies for this function handle, for A/B timing and tests; a
 * handle starts with every policy on.  "pair" = 0: keep the one-SM entry of the tcgen05 matmul on
 * grids that are even in x and y.  "tail_split" = 0: run every tile of the FFMA matmul whole.
 * "pdl" = 0: launch a coarsened kernel with an ordinary launch instead of programmatic stream serialisation
 * (the emitted kernels begin with griddepcontrol.wait, so the serialised form keeps stream order).
 * "tail_rounds" = r (1 to 8; 0 = the default: one, or two under basalt_rt_launch_gather): the stream units
 * that work the FFMA matmul's tail wave off come in r rounds of one unit per CTA slot.
 * "coarse_waves" = w > 0: launch a coarsened one-element-per-thread kernel on exactly w resident
 * waves instead of one loop trip per thread.  Unknown keys are refused (kind 4).  The state lives in
 * the handle: nothing here reads the process environment.  No counterpart in the reference. */
int basalt_rt_function_tune(basalt_rt_function *fn, const char *key, int value);
/* Kernels with bounded device-side waits (the tcgen05 matmul) own a device status word; this
 * reads it after synchronising: 0 = every wait was satisfied, non-zero = a wait gave up and the
 * output of that launch is not valid. No counterpart: the reference's kernels never wait. */
int basalt_rt_kernel_status(basalt_rt_function *fn, int32_t *out);
int basalt_rt_ctx_sync(basalt_rt_ctx *ctx);   /* cuCtxSynchronize (module.rs:120-121) */

/* Streams and events (no counterpart: ffi.rs:38-42 "no multi-stream support yet"). */
int basalt_rt_stream_create(basalt_rt_ctx *ctx, void **stream_out);
int basalt_rt_stream_destroy(basalt_rt_ctx *ctx, void *stream);
int basalt_rt_stream_sync(basalt_rt_ctx *ctx, void *stream);
int basalt_rt_event_create(basalt_rt_ctx *ctx, void **event_out);
int basalt_rt_event_destroy(basalt_rt_ctx *ctx, void *event);
int basalt_rt_event_record(basalt_rt_ctx *ctx, void *event, void *stream);
int basalt_rt_event_sync(basalt_rt_ctx *ctx, void *event);
int basalt_rt_event_elapsed_ms(basalt_rt_ctx *ctx, void *start, void *end, float *ms);

/* The reference's CPU launch ABI run on the device (crates/basalt-x86/src/oracle.rs:75-83,
 * examples/cpu_launch_*.c): host pointers in, results in host memory out. For each argument:
 * kind 0 = i32, 1 = i64, 2 = f32, 3 = f64 (value read from `value`), 4 = pointer read by the
 * kernel, 5 = pointer written, 6 = both (host address in `host`, extent in `bytes`). The call
 * takes device buffers (kept with the context between calls and reused by size), copies inputs,
 * launches ceil(nthreads/block) blocks of `block` threads (the reference's grid for a flat launch)
 * and copies outputs back.  Host buffers of 2 MiB or more that are not page-locked -- what a caller
 * of the reference's ABI passes -- are moved in chunks (4 MiB; 1 MiB below 32 MiB) by up to eight host threads through pinned
 * staging buffers, each thread feeding the copy engine on its own stream, instead of through the
 * driver's own pageable path; page-locked buffers (basalt_rt_host_alloc) are copied directly.  The
 * synchronous forms of basalt_rt_copy_from_host / basalt_rt_copy_to_host (stream NULL) do the same. */
typedef struct basalt_rt_arg {
    int kind;
    union { int32_t i32; int64_t i64; float f32; double f64; } value;
    void *host;
    size_t bytes;
} basalt_rt_arg;
int basalt_rt_cpu_launch(basalt_rt_ctx *ctx, basalt_rt_function *fn, const basalt_rt_arg *args, int nargs,
                         int64_t nthreads, uint32_t block);

/* Contiguous range [begin,end) of `total` units owned by `rank` of `nranks`, boundaries rounded
 * to multiples of `align` units. The grid-range sharding of the multi-GPU configurations. */
void basalt_rt_shard_range(uint64_t total, int nranks, int rank, uint64_t align, uint64_t *begin,
                           uint64_t *end);

/* NCCL over NVLink, one communicator rank per process (no counterpart in the reference). The id
 * made on rank 0 is distributed by the caller. */
int basalt_rt_comm_unique_id(char id_out[128]);
int basalt_rt_comm_init(basalt_rt_ctx *ctx, const char id[128], int nranks, int rank, basalt_rt_comm **out);
void basalt_rt_comm_destroy(basalt_rt_comm *comm);
/* ncclAllReduce(ncclInt32, ncclMax): combines the per-GPU partial maxima. */
int basalt_rt_allreduce_max_i32(basalt_rt_comm *comm, uint64_t send, uint64_t recv, size_t count, void *stream);
/* ncclAllGather of bytes_per_rank bytes: gathers the row-sharded matmul output. */
int basalt_rt_allgather(basalt_rt_comm *comm, uint64_t send, uint64_t recv, size_t bytes_per_rank, void *stream);

/* Whole-buffer peer mappings for the row-sharded matmuls, whose gather is overlapped with the
 * compute by pushing finished row bands into every peer's result buffer with the copy engines:
 * export a buffer allocated with basalt_rt_alloc as a 64-byte CUDA IPC handle, open another
 * process's handle (the returned address is valid on this context's device, for kernels and for
 * copies), close it again.  basalt_rt_copy_device_async is cuMemcpyDtoDAsync between any two such
 * addresses, basalt_rt_stream_wait_event orders one stream after an event recorded on another.
 * No counterpart in the reference (single GPU, synchronous copies only). */
int basalt_rt_ipc_export(const basalt_rt_buffer *buf, unsigned char handle_out[64]);
int basalt_rt_ipc_open(basalt_rt_ctx *ctx, const unsigned char handle[64], uint64_t *ptr_out);
int basalt_rt_ipc_close(basalt_rt_ctx *ctx, uint64_t ptr);
int basalt_rt_copy_device_async(basalt_rt_ctx *ctx, uint64_t dst, uint64_t src, size_t bytes, void *stream);
int basalt_rt_stream_wait_event(basalt_rt_ctx *ctx, void *stream, void *event);

/* Peer-memory exchange group: the sharded max_i32's allreduce without a library collective.  Each
 * rank creates a group (which allocates and zeroes its inbox), exports the inbox as a CUDA IPC
 * handle (64 bytes), receives every rank's handle through whatever channel the host program has
 * (torch.distributed in bench.py and the tests), and connects.  basalt_rt_peer_allreduce_max_i32
 * then launches basalt_k_peer_allreduce_max_i32 on `stream` with the next epoch (`reset`: store
 * reset_value into *partial after reading it).  `status` reads
 * the device word after synchronising: non-zero bits are ranks that did not answer within the
 * bound (2 s); a group that has reported a non-zero status must be destroyed and created again on
 * every rank (a late word matches no later epoch).  No counterpart in the reference (single GPU
 * only). */
typedef struct basalt_rt_peer_group basalt_rt_peer_group;
int basalt_rt_peer_group_create(basalt_rt_ctx *ctx, int nranks, int rank, basalt_rt_peer_group **out);
int basalt_rt_peer_group_handle(basalt_rt_peer_group *g, unsigned char handle_out[64]);
int basalt_rt_peer_group_connect(basalt_rt_peer_group *g, const unsigned char *handles, size_t nbytes);
int basalt_rt_peer_allreduce_max_i32(basalt_rt_peer_group *g, uint64_t partial, uint64_t result, int reset,
                                     int32_t reset_value, void *stream);
/* The whole sharded max_i32 step in one launch (basalt_k_max_i32_allreduce): reduction of the rank's
 * shard and the exchange, with the group's own running-maximum and ticket words. */
int basalt_rt_peer_max_i32(basalt_rt_peer_group *g, uint64_t shard, int64_t n, uint64_t result, void *stream);
int basalt_rt_peer_group_status(basalt_rt_peer_group *g, uint32_t *status_out);
int basalt_rt_peer_group_destroy(basalt_rt_peer_group *g);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* BASALT_B200_H */
