/*
 * flame_offload.h: C ABI of the B200 (sm_100a) activation offload/restore path.
 *
 * Plain C, no C++ or framework types: every argument is a pointer, a size or a
 * scalar.  All device pointers are raw CUDA device addresses, every `stream`
 * is a cudaStream_t passed as void* (NULL = the legacy default stream).  No
 * entry point calls cudaDeviceSynchronize, throws, or aborts.
 *
 * Two return conventions coexist because the reference project has two:
 *   - `int` that is 0 on success and otherwise the cudaError_t value
 *     (the pinned_host.cu / fp8_quant.cu family);
 *   - FlameOffloadStatus (the FlameCudaStatus family of
 *     cuda/include/flame_cuda_status.h, extended by two codes).
 *
 * Each declaration names the reference interface (file:line inside the
 * reference project) that it replaces or extends.
 */
#ifndef FLAME_OFFLOAD_H_
#define FLAME_OFFLOAD_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Same numbering as FlameCudaStatus (cuda/include/flame_cuda_status.h:7-12,
 * mapped to Rust errors at src/cuda_ops_ffi.rs:591-599); 4 and 5 are new.
 * STATE corresponds to the reference's Error::InvalidOperation (pool full,
 * stale epoch, slot out of range, slot not in the Pushed state:
 * src/activation_offload.rs:494-499, 620-641). */
typedef enum {
  FLAME_OFFLOAD_OK = 0,
  FLAME_OFFLOAD_ERR_INVALID = 1,
  FLAME_OFFLOAD_ERR_UNSUPPORTED = 2,
  FLAME_OFFLOAD_ERR_CUDA = 3,
  FLAME_OFFLOAD_ERR_TIMEOUT = 4,
  FLAME_OFFLOAD_ERR_STATE = 5
} FlameOffloadStatus;

/* Text of the last error raised on the calling thread ("" if none). */
const char* flame_offload_last_error(void);

/* ------------------------------------------------------------------------
 * 1. Pinned host memory and async copies: signatures kept exactly.
 *    Replaces src/cuda/pinned_host.cu:4-45 (declared src/cuda/ffi.rs:83-94).
 * ---------------------------------------------------------------------- */
void* flame_cuda_alloc_pinned_host(size_t size, unsigned int flags); /* NULL on failure */
int flame_cuda_free_pinned_host(void* ptr);
/* kind: 1 = H2D, 2 = D2H, 3 = D2D, anything else = cudaMemcpyDefault */
int flame_cuda_memcpy_async(void* dst, const void* src, size_t bytes, int kind, void* stream);
int flame_cuda_host_register(void* ptr, size_t bytes, unsigned int flags);
int flame_cuda_host_unregister(void* ptr);

/* Replaces src/ffi/cuda_ffi.c:90-109 (impl cuda/src/flame_cuda_common.cu:131-165):
 * NULL pointers or bytes == 0 give ERR_INVALID. */
FlameOffloadStatus flame_h2d_async(void* dst_device, const void* src_host, uint64_t bytes, void* stream);
FlameOffloadStatus flame_d2h_async(void* dst_host, const void* src_device, uint64_t bytes, void* stream);
FlameOffloadStatus flame_d2d_async(void* dst_device, const void* src_device, uint64_t bytes, void* stream);

/* ------------------------------------------------------------------------
 * 2. Element-wise FP8 E4M3 with a caller-supplied scale: signatures kept.
 *    Replaces src/cuda/fp8_quant.cu:74-93 and src/cuda/fp8_dequant.cu:41-59
 *    (declared src/cuda/ffi.rs:546-564, src/activation_offload.rs:99-115).
 *    out[i] = enc(bf16_to_f32(in[i]) * inv_scale);  out[i] = bf16(dec(in[i]) * scale)
 *    with the reference's own encoder/decoder arithmetic, bit for bit, under
 *    IEEE (non flush-to-zero) float semantics.  n == 0 returns 0 at once.
 * ---------------------------------------------------------------------- */
int flame_bf16_to_fp8(const void* input_bf16, void* output_u8, float inv_scale, size_t n_elements, void* stream);
int flame_fp8_to_bf16(const void* input_u8, void* output_bf16, float scale, size_t n_elements, void* stream);

/* FP8 E4M3 weights with the transpose built in: signature kept.
 * Replaces src/cuda/fused_dequant_transpose.cu:104-126 (declared src/cuda/ffi.rs, called from
 * src/ops/fused_inference.rs:140-175): input [M, N] row-major FP8 bytes, output [N, M] row-major BF16,
 * out[n][m] = bf16_rn(dec(in[m][n]) * scale) with that file's decoder (sub-normals, exponent 15 with a zero
 * mantissa = 256, exponent 15 with any other mantissa = NaN), bit for bit under IEEE float semantics.
 * M == 0 or N == 0 returns 0 at once.  M % 8 == 0, N % 8 == 0, an 8-byte aligned input and a 16-byte aligned
 * output take the fast kernel. */
int flame_fused_dequant_transpose_bf16(const void* input_fp8, void* output_bf16, float scale, int M, int N, void* stream);

/* The same for several weights in one launch (new): what a block of a model needs expanded once its bytes have
 * arrived.  The reference calls its kernel once per weight (src/ops/fused_inference.rs:140-175); here the caller makes
 * one call, and the library one launch, for a block's four to eight weights.  Every job has the meaning of one
 * flame_fused_dequant_transpose_bf16 call; jobs with M == 0 or N == 0 are skipped; a job that misses the fast
 * kernel's conditions gets a launch of its own.  Outputs must not overlap each other or any input.
 * count <= 0 returns 0 at once. */
typedef struct FlameWeightJob {
  const void* input_fp8;   /* [M, N] row-major E4M3 codes */
  void* output_bf16;       /* [N, M] row-major BF16 */
  float scale;
  int M;
  int N;
  int reserved;            /* 0 */
} FlameWeightJob;          /* 32 bytes */
int flame_fused_dequant_transpose_bf16_multi(const FlameWeightJob* jobs, int count, void* stream);

/* ------------------------------------------------------------------------
 * 3. Per-128-element-block codecs (new; they take the place of the two calls
 *    above inside push/pull, src/activation_offload.rs:543-579 and 678-700).
 *
 *    Blocks are consecutive runs of 128 elements of the flat tensor; a short
 *    last block uses only its real elements.  scales[b] is fp32.
 *      int8: scale = absmax/127; code = rne(x / scale) in [-127,127]
 *            (int8 formula of src/sage_attention.rs:524-541); absmax == 0
 *            gives scale 0 and codes 0.
 *      fp8 : scale = absmax/448; code = enc(x * (1/scale)) with the encoder of
 *            src/cuda/fp8_quant.cu:19-57; absmax == 0 gives scale 0, codes 0.
 *    Dequantise: out = bf16_rne(float(code) * scale) / bf16_rne(dec(code) * scale).
 *    Returns 0 or a cudaError_t value; cudaErrorInvalidValue (1) for NULL
 *    pointers with n > 0.  Any pointer alignment is accepted (32-byte aligned
 *    BF16 buffers and 16-byte aligned code/scale buffers take the fast kernels).
 *    Each call is a few kernel launches on `stream` and nothing else (no
 *    allocation, no synchronisation), so the calls can be recorded in a CUDA
 *    graph; call each entry point once on the device before the capture, so
 *    that the runtime has loaded the kernels.  The fast kernels (and the FP8
 *    weight kernel above) are launched with programmatic stream serialisation
 *    and wait inside the kernel for whatever precedes them in the stream, so
 *    that one of them directly behind another starts without a launch's
 *    start-up time; stream order and results are unchanged.  The environment
 *    variable FLAME_ACT_PDL=0 makes them plain launches.
 * ---------------------------------------------------------------------- */
#define FLAME_ACT_BLOCK 128
#define FLAME_ACT_INT8_MUL_INV 1u /* int8: code = rne(x * (1/scale)) instead of the division */
#define FLAME_ACT_FP8_OCP 1u      /* fp8: OCP round-to-nearest-even, saturating encoder (not the reference's) */
#define FLAME_ACT_STAGED_STORES 2u /* compress: each warp collects its 1024 codes and 8 scales of a tile in shared memory and
                                      one lane writes them with two bulk asynchronous copies instead of per-lane stores
                                      (warp-level synchronisation only); same results */

int flame_act_quant_int8_b128(const void* in_bf16, void* codes_i8, void* scales_f32, size_t n, unsigned int flags, void* stream);
int flame_act_dequant_int8_b128(const void* codes_i8, const void* scales_f32, void* out_bf16, size_t n, void* stream);
int flame_act_quant_fp8_b128(const void* in_bf16, void* codes_u8, void* scales_f32, size_t n, unsigned int flags, void* stream);
int flame_act_dequant_fp8_b128(const void* codes_u8, const void* scales_f32, void* out_bf16, size_t n, void* stream);

/* Producers with the compress step built in: the tensor a checkpointed block saves is written once, together
 * with its codes and scales, and no compress launch reads it again.  The codes and scales are bit for bit what
 * flame_act_quant_*_b128 gives for the BF16 tensor these kernels write (y) or read (gate_up).
 * codec: 0 (BF16 output only), FLAME_OFFLOAD_COMPRESSION_INT8_B128 or _FP8_B128; flags as for the quantisers.
 *
 * RMSNorm, the arithmetic of src/cuda/fused_rms_norm.cu:26-80: y = bf16((x * rsqrt(mean(x^2) + eps)) * weight), fp32
 * inside; x, y [rows, cols], weight [cols], cols % 128 == 0, cols <= 16384; codes [rows*cols], scales [rows*cols/128]
 * describe y; rstd_f32 [rows] (may be NULL) receives rsqrt(mean(x^2) + eps) for a backward pass that works from y. */
int flame_act_rmsnorm_quant_b128(const void* x_bf16, const void* weight_bf16, void* y_bf16, void* codes_u8, void* scales_f32,
                                 void* rstd_f32, size_t rows, size_t cols, float eps, int codec, unsigned int flags, void* stream);
/* SwiGLU: gate_up [rows, 2*hidden] = gate columns then up columns, h [rows, hidden] = bf16(silu(gate) * up), hidden % 128
 * == 0; codes [rows*2*hidden] and scales describe gate_up, the pair the backward pass needs
 * (Op::FusedSwiGLU{gate, up}, src/autograd.rs:326-331). */
int flame_act_swiglu_quant_b128(const void* gate_up_bf16, void* h_bf16, void* codes_u8, void* scales_f32, size_t rows, size_t hidden,
                                int codec, unsigned int flags, void* stream);

/* Several tensors in one launch: the saved activations of a checkpointed block
 * are pushed together (the loop at src/autograd.rs:1714-1741), and one launch over
 * all of them avoids a launch gap and a ragged last wave per tensor.  Results are
 * identical to calling the single-tensor entry points one by one. */
typedef struct {
  void* bf16;   /* BF16 tensor: source of quantise, destination of dequantise */
  void* codes;  /* n bytes */
  void* scales; /* ceil(n/128) floats */
  size_t n;
} FlameActTensor;
/* codec: FLAME_OFFLOAD_COMPRESSION_INT8_B128 or _FP8_B128 */
int flame_act_quant_b128_multi(int codec, const FlameActTensor* tensors, size_t count, unsigned int flags, void* stream);
int flame_act_dequant_b128_multi(int codec, const FlameActTensor* tensors, size_t count, void* stream);

/* Packed layout of one compressed tensor or chunk in one buffer:
 * codes[n] | zero padding up to a 256-byte boundary | scales[ceil(n/128)]. */
size_t flame_act_packed_scales_offset(size_t n);
size_t flame_act_packed_bytes(size_t n);

/* Compress `n` BF16 elements on the device and deliver the packed result
 * (layout above, flame_act_packed_bytes(n) bytes) to `packed_out`, which may be
 * pinned host memory or device memory, WITHOUT allocating anything: no
 * cudaMalloc, cudaFree or other allocating call is made.  (No counterpart in the
 * reference, whose pool allocates its staging buffers up front,
 * src/activation_offload.rs:401-407.)
 *
 * For callers that cannot allocate at the moment they need to spill: an
 * out-of-memory handler freeing device memory by moving an activation out, or
 * a step loop with a fixed memory plan in which cudaMalloc/cudaFree would stall
 * the device or fail.  The device staging it needs is a fixed array inside the
 * library: every GPU that uses the library holds about 8.3 MiB of it until the
 * process exits.
 *
 *   - The CUDA runtime loads a library's kernels and static device arrays when
 *     they are first used on a device, not when the library is opened, and that
 *     loading itself takes device memory.  A caller that wants the no-allocation
 *     property at the moment of need therefore makes one small warm-up call per
 *     device at start-up, for each codec it will use and for both a 32-byte
 *     aligned and an unaligned input (they run different kernels), while
 *     memory is still available.  After that, a call takes no device memory.
 *   - n may be at most FLAME_ACT_NOALLOC_MAX_ELEMS; larger tensors are refused
 *     with cudaErrorInvalidValue (1) and a message in flame_offload_last_error().
 *   - codec is FLAME_OFFLOAD_COMPRESSION_INT8_B128 or _FP8_B128; flags as for
 *     the quantise entry points.  Results are identical to those entry points.
 *   - The first call on each device also looks up the array's device address
 *     (cudaGetSymbolAddress); make that first call before starting any stream
 *     capture on that device.
 *   - All calls share the one array.  Calls on the same stream are ordered;
 *     calls whose GPU work can overlap (different streams) race on it and must
 *     be ordered by the caller.  The result is complete when `stream` reaches
 *     the end of the call's work. */
#define FLAME_ACT_NOALLOC_MAX_ELEMS ((size_t)8 << 20)
int flame_act_offload_packed_noalloc(const void* in_bf16, void* packed_out, size_t n, int codec, unsigned int flags, void* stream);

/* Limits the number of thread blocks the codec kernels launch on the current
 * device (0 = default: a multiple of the SM count).  Returns the old value. */
int flame_act_set_max_ctas(int max_ctas);

/* Tuning hook: the compress kernel exists in three forms that write the same bytes (0: load, encode, store with
 * five resident thread blocks per SM; 1: software-pipelined loads, four resident blocks; 2: as 0 with four
 * resident blocks).  form 0..2 forces one for both codecs, anything else restores the per-codec defaults (also
 * settable once per process by the environment variable FLAME_ACT_COMPRESS_FORM).  Returns the previous
 * override, -1 if none.  No counterpart in the reference. */
int flame_act_set_compress_form(int form);

/* Inspection of launch decisions (no counterpart in the reference, whose kernels use a fixed
 * (n + 255) / 256 grid, src/cuda/fp8_quant.cu:84-88).  flame_act_last_launch: grid, resident thread
 * blocks per SM the grid was sized for, tiles per block and kernel form (0..2, +4 with staged stores)
 * of the calling thread's most recent fast-path compress or dequantise launch.
 * flame_act_query_resident_blocks: a fresh occupancy query on the current device for the kernel a
 * (codec, flags, form) selects; form < 0 = the codec's default form; compress 0 = the dequantise
 * kernel.  Returns -1 on error. */
typedef struct {
  int32_t grid, resident_per_sm, tiles_per_block, form;
} FlameActLaunchInfo;
void flame_act_last_launch(FlameActLaunchInfo* out);
int flame_act_query_resident_blocks(int codec, unsigned int flags, int form, int compress);

/* ------------------------------------------------------------------------
 * 4. Activation offload pool.
 *    Mirrors ActivationOffloadPool (src/activation_offload.rs:323-760): same
 *    slot state machine, LIFO free stack, epoch-stamped handles and error
 *    cases.  Underneath: one pinned slab carved into chunks, a chunked
 *    double-buffered pipeline on dedicated codec / D2H / H2D streams, and
 *    restore straight into a caller-provided destination.
 * ---------------------------------------------------------------------- */
typedef struct FlameOffloadPool FlameOffloadPool;

/* OffloadCompression (src/activation_offload.rs:89-96) plus the two block codecs. */
enum {
  FLAME_OFFLOAD_COMPRESSION_NONE = 0,
  FLAME_OFFLOAD_COMPRESSION_FP8 = 1,       /* reference mode: fixed per-tensor scale 8/448 */
  FLAME_OFFLOAD_COMPRESSION_INT8_B128 = 2,
  FLAME_OFFLOAD_COMPRESSION_FP8_B128 = 3
};

/* DType tags accepted by push (src/activation_offload.rs:467-476). */
enum { FLAME_OFFLOAD_DTYPE_BF16 = 0, FLAME_OFFLOAD_DTYPE_F32 = 1 };

/* OffloadHandle (src/activation_offload.rs:292-303): a plain copyable value. */
typedef struct {
  uint64_t slot;
  uint64_t epoch;
} FlameOffloadHandle;

typedef struct {
  uint32_t struct_size;       /* sizeof(FlameOffloadPoolConfig); 0-filled fields take defaults */
  int32_t device;             /* CUDA ordinal; -1 = current device */
  uint64_t chunk_bytes;       /* pipeline chunk in source (BF16/F32) bytes; default 16 MiB; multiple of 64 KiB */
  uint32_t staging_tiles;     /* device staging tiles per direction for the compressed modes; default 2 */
  uint32_t codec_flags;       /* FLAME_ACT_* flags passed to the block codecs */
  uint64_t host_budget_bytes; /* pinned bytes to hold; 0 = num_slots * stored size of max_bytes */
  uint32_t host_alloc_flags;  /* cudaHostAlloc flags; default 0 (never write-combined: the host reads it back) */
  int32_t codec_max_ctas;     /* thread blocks per codec launch; 0 = default */
  int32_t numa_node;          /* bind the slab to this NUMA node with mbind(); -1 = leave to first touch */
  uint32_t tile_chunks;       /* chunks per staging tile = per codec kernel launch; default 8 */
  uint64_t d2h_piece_bytes;   /* a chunk's device-to-host copy is issued in pieces of this size; 0 = whole chunk.
                                 A copy engine that saturates the link slows concurrent HBM-bound kernels by
                                 50 % and more; 1-2 MiB pieces leave gaps that cut this to ~10-20 % at ~85 %
                                 of the copy rate.  Use small pieces when offload overlaps training compute. */
  uint64_t h2d_piece_bytes;   /* the same for host-to-device copies; 0 = whole chunk */
  uint64_t deferred_inflight_bytes; /* 0 = push() enqueues its copies at once (the reference's behaviour).  > 0 = deferred
                                 offload: push() only queues the tensor; a thread owned by the pool enqueues
                                 compress + device-to-host work in push order while less than this many pinned
                                 bytes are in flight.  A tensor whose turn has not come when backward needs it
                                 is still on the device: flame_offload_pool_cancel() takes it out of the queue
                                 and the caller uses the source as it is, so the link never holds backward up
                                 with round trips that free no memory.  About one block's stored bytes
                                 (1-4 x 100 MB) keeps the link busy. */
  uint32_t collect_timing;    /* non-zero: time every offload, every restore and every wait for a restore with a pair of
                                 timing-enabled events and report the sums in FlameOffloadStats (the reference traces
                                 behind environment switches, src/autograd.rs:1086-1089, 1501-1547).  Off by default:
                                 two more event records per push and four per pull. */
  uint32_t reserved0;
} FlameOffloadPoolConfig;

typedef struct {
  uint64_t pushes, pulls;
  uint64_t bytes_logical_out, bytes_logical_in; /* BF16/F32 bytes offloaded / restored */
  uint64_t bytes_link_out, bytes_link_in;       /* bytes that crossed the host link */
  uint64_t chunks_out, chunks_in;
  uint64_t codec_launches;                      /* compress + dequantise kernel launches */
  uint64_t host_chunks_total, host_chunks_free;
  uint64_t push_rejected_full;                  /* pushes refused: no slot or no pinned chunk left */
  uint64_t pushes_cancelled;                    /* deferred pushes taken back before their copies were enqueued */
  uint64_t pushes_queued;                       /* deferred pushes waiting for their turn right now */
  /* With FlameOffloadPoolConfig.collect_timing, device time in microseconds, summed over the spans the device has
   * finished when the statistics are read (spans_pending are still running):
   *   offload_span_us  per offload, from the moment the device-to-host stream has the tensor (or its first compressed
   *                    tile) in front of it to the end of its last copy: link time plus what the stream waited for
   *                    later tiles to be compressed;
   *   restore_span_us  per restore, from the moment the host-to-device stream may start (the offload has finished) to
   *                    the end of its last copy;
   *   ready_wait_us    per wait for a restore (pull_into without DEFER_WAIT, wait_ready), from the moment the caller's
   *                    stream reaches the wait to the moment it passes: what the restores cost the stream that
   *                    consumes them. */
  uint64_t offload_span_us, restore_span_us, ready_wait_us;
  uint64_t spans_timed, spans_pending;
} FlameOffloadStats;

/* new(device, num_slots, max_bytes, compression): src/activation_offload.rs:365-427.
 * cfg may be NULL.  Returns NULL on failure (see flame_offload_last_error). */
FlameOffloadPool* flame_offload_pool_create(size_t num_slots, size_t max_bytes, int compression, const FlameOffloadPoolConfig* cfg);
/* Waits (bounded, 30 s) for the pool's own streams, then frees everything. */
void flame_offload_pool_destroy(FlameOffloadPool* pool);

/* Accessors: src/activation_offload.rs:429-455. */
size_t flame_offload_pool_num_slots(const FlameOffloadPool* pool);
size_t flame_offload_pool_slot_bytes(const FlameOffloadPool* pool);
size_t flame_offload_pool_host_bytes(const FlameOffloadPool* pool);
size_t flame_offload_pool_in_flight(const FlameOffloadPool* pool);
int flame_offload_pool_compression(const FlameOffloadPool* pool);

/* push(&tensor): src/activation_offload.rs:465-611.  `src_device` must be the
 * first element of a contiguous tensor of `numel` elements.  Work already
 * submitted to `compute_stream` is ordered before the pool reads the source.
 * Never blocks the host.  The caller must keep the source alive until
 * flame_offload_pool_source_released() reports 1 (the reference holds it until
 * pull; src/activation_offload.rs:600-605). */
FlameOffloadStatus flame_offload_pool_push(FlameOffloadPool* pool, const void* src_device, size_t numel, int dtype, void* compute_stream, FlameOffloadHandle* out_handle);

/* pull(handle): src/activation_offload.rs:619-731, but into the caller's
 * buffer (`dst_bytes` >= the tensor's byte size).  Work already submitted to
 * `compute_stream` is ordered before the first write into dst.  Unless
 * FLAME_OFFLOAD_PULL_DEFER_WAIT is set, `compute_stream` is made to wait for
 * the restore before returning (src/activation_offload.rs:714-715).  The slot
 * returns to Idle and to the top of the free stack, unless FLAME_OFFLOAD_PULL_KEEP
 * is set: then the slot stays Pushed with its pinned copy intact and the same
 * handle can be restored again (block weights streamed in every step, the
 * pattern of the pinned staging helpers in src/pinned.rs:320-401; the reference's
 * pool itself has no non-consuming pull). */
#define FLAME_OFFLOAD_PULL_DEFER_WAIT 1u
#define FLAME_OFFLOAD_PULL_KEEP 2u
FlameOffloadStatus flame_offload_pool_pull_into(FlameOffloadPool* pool, FlameOffloadHandle handle, void* dst_device, size_t dst_bytes, void* compute_stream, unsigned int flags);
/* prefetch(handle): the restore is started now and nothing waits for it yet; the consumer calls
 * flame_offload_pool_wait_ready(pool, handle.slot, stream) before its first read.  Same as pull_into with
 * FLAME_OFFLOAD_PULL_DEFER_WAIT; the reference pulls just in time (src/autograd.rs:2470-2479). */
FlameOffloadStatus flame_offload_pool_prefetch(FlameOffloadPool* pool, FlameOffloadHandle handle, void* dst_device, size_t dst_bytes, void* compute_stream);
/* Makes `stream` wait for the most recent restore issued from `slot`. */
FlameOffloadStatus flame_offload_pool_wait_ready(FlameOffloadPool* pool, size_t slot, void* stream);

/* push of a tensor that is already compressed on the device (by the producers above, or by flame_act_quant_*_b128):
 * `codes_device` [numel] and `scales_device` [ceil(numel/128)] go to the pinned slab as they are, no compress launch.
 * The pool must be in the matching block mode (INT8_B128 / FP8_B128); numel counts BF16 elements; both buffers
 * must stay alive until flame_offload_pool_source_released() reports 1.  pull_into restores BF16 as usual. */
FlameOffloadStatus flame_offload_pool_push_packed(FlameOffloadPool* pool, const void* codes_device, const void* scales_device, size_t numel, void* compute_stream, FlameOffloadHandle* out_handle);

/* The counterpart of push_packed: restores the compressed form itself, `numel` codes into `codes_device` and
 * ceil(numel/128) scales into `scales_device` (no staging tile, no dequantise launch), so that the caller can
 * expand several tensors with one flame_act_dequant_b128_multi launch when it needs them.  Flags and ordering as
 * for pull_into; the pool must be in a per-128-block mode. */
FlameOffloadStatus flame_offload_pool_pull_packed(FlameOffloadPool* pool, FlameOffloadHandle handle, void* codes_device, void* scales_device, void* compute_stream, unsigned int flags);

/* Deferred offload only (deferred_inflight_bytes > 0).  1: the tensor was still waiting for its turn; its slot
 * and chunks are free again, nothing was or will be read from the source, which the caller goes on using.
 * 0: its copies are already enqueued (or the pool is not deferred): restore it with pull_into as usual.
 * Negative: -FlameOffloadStatus (stale or invalid handle). */
int flame_offload_pool_cancel(FlameOffloadPool* pool, FlameOffloadHandle handle);
/* Deferred offload only: while `on` is non-zero the pool's thread enqueues nothing new (backward has begun:
 * what is still queued is about to be needed and will be cancelled); tensors pulled while queued are still
 * enqueued at once.  0 resumes. */
FlameOffloadStatus flame_offload_pool_hold(FlameOffloadPool* pool, int on);
/* Deferred offload only: the hold begins when the work submitted to `stream` so far has finished on the device.
 * The host runs ahead of the device, so "backward has begun" on the host says little; called when the host
 * starts backward, this stops new offloads when the DEVICE has finished the forward pass (after which sending
 * tensors out no longer lowers the peak), while tensors the host reaches earlier are cancelled as usual.
 * flame_offload_pool_hold(pool, 0) ends it. */
FlameOffloadStatus flame_offload_pool_hold_after(FlameOffloadPool* pool, void* stream);

/* Gives the slot of `handle` back without restoring it (the reference releases
 * the slots of an abandoned block by pulling every handle,
 * src/autograd.rs:1742-1769; this does the same bookkeeping without the copy). */
FlameOffloadStatus flame_offload_pool_discard(FlameOffloadPool* pool, FlameOffloadHandle handle);

/* clear(): src/activation_offload.rs:742-760.  Does not synchronise. */
FlameOffloadStatus flame_offload_pool_clear(FlameOffloadPool* pool);

/* 1 when the device-to-host copy of `handle` has finished reading the source
 * tensor (it may be freed), 0 while it is still being read, negative
 * FlameOffloadStatus on a stale or invalid handle. */
int flame_offload_pool_source_released(FlameOffloadPool* pool, FlameOffloadHandle handle);

/* Metadata captured at push (SlotMeta, src/activation_offload.rs:269-281). */
typedef struct {
  uint64_t numel;
  int32_t dtype;
  int32_t compression;
  uint64_t bytes;        /* logical bytes */
  uint64_t stored_bytes; /* pinned bytes used, scales and padding included */
  uint64_t chunks;
} FlameOffloadSlotInfo;
FlameOffloadStatus flame_offload_pool_slot_info(FlameOffloadPool* pool, FlameOffloadHandle handle, FlameOffloadSlotInfo* out);

/* Polls the pool's streams until idle or until timeout_s elapses
 * (ERR_TIMEOUT).  Never waits unboundedly. */
FlameOffloadStatus flame_offload_pool_synchronize(FlameOffloadPool* pool, double timeout_s);

/* Test / inspection hook: after the offload of `handle` has completed, gather
 * what is stored in pinned memory into host arrays in canonical order.
 * Compressed modes: codes_out[numel] and scales_out[ceil(numel/128)] (legacy
 * FP8: scales_out[0] = the fixed scale).  Uncompressed: codes_out[bytes]. */
FlameOffloadStatus flame_offload_pool_read_slot(FlameOffloadPool* pool, FlameOffloadHandle handle, void* codes_out, void* scales_out, double timeout_s);

FlameOffloadStatus flame_offload_pool_stats(const FlameOffloadPool* pool, FlameOffloadStats* out);

/* Host-side fault injection for tests: the `countdown`-th next call of the
 * named kind fails with an error code instead of reaching CUDA.  Nothing is
 * ever injected on the device. */
enum { FLAME_OFFLOAD_FAULT_NONE = 0, FLAME_OFFLOAD_FAULT_MEMCPY = 1, FLAME_OFFLOAD_FAULT_KERNEL = 2, FLAME_OFFLOAD_FAULT_HOST_ALLOC = 3 };
void flame_offload_inject_fault(int kind, int countdown);

/* ------------------------------------------------------------------------
 * 5. PinnedPool: size-class cache of pinned buffers.
 *    Mirrors src/pinned_pool.rs:21-99 (8 MiB classes, max_cached_bytes cap).
 * ---------------------------------------------------------------------- */
typedef struct FlamePinnedPool FlamePinnedPool;
FlamePinnedPool* flame_pinned_pool_create(unsigned int alloc_flags, size_t max_cached_bytes);
void flame_pinned_pool_destroy(FlamePinnedPool* pool);
/* checkout(min_bytes): smallest cached buffer with capacity >= round_up(min_bytes), else a fresh one. */
FlameOffloadStatus flame_pinned_pool_checkout(FlamePinnedPool* pool, size_t min_bytes, void** out_ptr, size_t* out_capacity);
/* checkin(buf): cached if it fits under max_cached_bytes, otherwise freed. */
FlameOffloadStatus flame_pinned_pool_checkin(FlamePinnedPool* pool, void* ptr, size_t capacity);
void flame_pinned_pool_stats(const FlamePinnedPool* pool, size_t* cached_bytes, size_t* cached_buffers);

/* ------------------------------------------------------------------------
 * 6. Bandwidth probes and the recompute-vs-offload policy.
 *    Takes the seat of CheckpointPolicy::Adaptive
 *    (src/gradient_checkpointing.rs:70-74, 201-232) and of the fixed rule
 *    "offload every BF16 requires_grad saved tensor" (src/autograd.rs:1721-1725).
 * ---------------------------------------------------------------------- */
typedef struct {
  double d2h_gbs, h2d_gbs;       /* pinned <-> device copy rate, GB/s */
  double hbm_copy_gbs;           /* device-to-device copy, read+write bytes per second */
  double quant_gbs, dequant_gbs; /* int8 block codec, algorithmic bytes per second */
} FlameLinkProbe;
/* Measures on the current device with CUDA events; `bytes` per transfer (0 = 256 MiB). */
FlameOffloadStatus flame_offload_probe(size_t bytes, int reps, FlameLinkProbe* out);

enum { FLAME_POLICY_RESIDENT = 0, FLAME_POLICY_OFFLOAD_BF16 = 1, FLAME_POLICY_OFFLOAD_INT8 = 2, FLAME_POLICY_OFFLOAD_FP8 = 3, FLAME_POLICY_RECOMPUTE = 4 };

typedef struct {
  uint64_t bytes;          /* BF16 bytes of the saved tensor */
  double recompute_ms;     /* time to recompute it in backward; < 0 = cannot be recomputed */
  int32_t group;           /* checkpoint block index in forward order */
  int32_t allow_lossy;     /* 1 = int8/fp8 allowed */
} FlamePolicyTensor;

typedef struct {
  double d2h_gbs, h2d_gbs;      /* from the probe, for this replica count */
  double fwd_ms, bwd_ms;        /* compute time of one step that copies can hide behind */
  uint64_t device_budget_bytes; /* activation bytes that may stay resident */
  int32_t lossy_codec;          /* FLAME_POLICY_OFFLOAD_INT8 or _FP8 */
  double link_utilisation;      /* fraction of fwd/bwd time the link may be busy; default 0.9 */
  double interference;          /* plan_blocks: extra compute time per unit of time a copy engine is busy beside it
                                   (copies slow HBM-bound kernels, see FlameOffloadPoolConfig.d2h_piece_bytes);
                                   ~0.1 measured on a B200 DiT step with 2 MiB pieces; 0 = ignore */
  double overhead_cap_ms;       /* plan_blocks: 0 = least estimated step time within device_budget_bytes (above).
                                   > 0 = the other way round: keep as few bytes resident as possible while the
                                   estimated extra step time (stalls + recompute + interference) stays at or under
                                   this many milliseconds; device_budget_bytes is then not consulted and the plan
                                   reports the resident bytes it ends with.  This is the mode for a link whose rate
                                   depends on how many replicas share it: the same cap gives a smaller offload on a
                                   slower link instead of a stalled backward pass. */
} FlamePolicyInput;

/* Deterministic for given inputs.  decisions[i] receives a FLAME_POLICY_* value. */
FlameOffloadStatus flame_offload_policy_plan(const FlamePolicyInput* in, const FlamePolicyTensor* tensors, size_t n, int32_t* decisions, double* est_overhead_ms);

/* Block-level plan for a stack of G checkpointed blocks run in order and
 * back-propagated in reverse.  Simulates the two FIFO copy queues against the
 * compute timeline: block g's saved bytes can start D2H when its forward ends,
 * must be back on the device when its backward starts, and a restore cannot
 * start before its own offload has finished.  Searches over how many trailing
 * blocks stay resident (within device_budget_bytes) and how many leading
 * blocks are recomputed instead, and returns the plan with the least estimated
 * step time (ties: fewest resident bytes); with overhead_cap_ms > 0 it returns
 * instead the plan with the fewest resident bytes whose estimate is under the
 * cap (all blocks resident always is).  Deterministic. */
typedef struct {
  uint64_t saved_bytes; /* BF16 bytes the block saves for backward */
  double fwd_ms;        /* forward time of the block (= its recompute cost) */
  double bwd_ms;        /* backward time of the block */
} FlamePolicyBlock;

typedef struct {
  double est_stall_ms;     /* backward waiting for restores, summed */
  double est_recompute_ms; /* forward re-runs inside backward */
  uint64_t resident_bytes; /* activation bytes kept on the device */
  uint64_t link_bytes;     /* payload per direction per step */
  double est_interference_ms; /* compute slowed by concurrent copies */
} FlamePolicyBlockPlan;

FlameOffloadStatus flame_offload_policy_plan_blocks(const FlamePolicyInput* in, const FlamePolicyBlock* blocks, size_t n, int offload_decision, int32_t* decisions, FlamePolicyBlockPlan* out);

/* ------------------------------------------------------------------------
 * 7. Restore arena: destinations for pull_into() out of one range reserved at
 *    set-up.  Replaces the fresh tensor of every pull
 *    (src/activation_offload.rs:655); the model is the reference's stream-keyed
 *    arena (src/staging.rs:219-297: arena_alloc, arena_record_and_release,
 *    arena_reset, arena_stats).
 *
 *    The arena is host bookkeeping over [base, base+bytes), memory the caller
 *    allocated once and keeps alive.  It belongs to ONE stream: every use of a
 *    region is queued on that stream (or ordered with it, as pull_into orders
 *    the pool's copies when it is given that stream), and release() is called
 *    after the last use has been queued.  Space is handed out in ring order;
 *    releases may arrive in any order and space returns when the oldest (or
 *    newest) regions have been released.  No call here touches CUDA.
 * ---------------------------------------------------------------------- */
typedef struct FlameRestoreArena FlameRestoreArena;
typedef struct {
  uint64_t capacity_bytes, in_use_bytes, peak_in_use_bytes;
  uint64_t allocs, releases, rejected, resets, live_regions;
} FlameRestoreArenaStats;
/* alignment: power of two, 0 = 256.  NULL on bad arguments. */
FlameRestoreArena* flame_restore_arena_create(void* base_device, size_t bytes, size_t alignment);
void flame_restore_arena_destroy(FlameRestoreArena* arena);
/* FLAME_OFFLOAD_ERR_STATE when no released space of that size is next in the ring (the caller falls back to its
 * own allocator); FLAME_OFFLOAD_ERR_INVALID when `bytes` is 0 or larger than the arena. */
FlameOffloadStatus flame_restore_arena_alloc(FlameRestoreArena* arena, size_t bytes, void** out_ptr, uint64_t* out_ticket);
FlameOffloadStatus flame_restore_arena_release(FlameRestoreArena* arena, uint64_t ticket);
/* Forgets every region (arena_reset, src/staging.rs:270): tickets handed out before are no longer valid. */
FlameOffloadStatus flame_restore_arena_reset(FlameRestoreArena* arena);
FlameOffloadStatus flame_restore_arena_stats(const FlameRestoreArena* arena, FlameRestoreArenaStats* out);

#ifdef __cplusplus
}
#endif
#endif /* FLAME_OFFLOAD_H_ */
