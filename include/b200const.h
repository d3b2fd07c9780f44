/*
 * b200const.h -- C ABI of the B200 constant-folding shim.
 *
 * This is the boundary a host compiler binds to in order to run the
 * vpux::Const::ContentAttr transformation chain (constant folding of weight
 * tensors) and the weight-compression codec on an NVIDIA B200 (sm_100a).
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, never
 * throws, and returns 0 on success or a negative B200C_ERR_* code.  The text of
 * the error (the message the reference would have put into VPUX_THROW) is kept
 * per calling thread and read with b200c_last_error().
 *
 * There is no CPU implementation behind these calls: when no CUDA device is
 * usable every compute entry point fails with B200C_ERR_CUDA.
 *
 * Reference interfaces are cited by their path inside openvinotoolkit/npu_plugin.
 */
#ifndef B200CONST_H_
#define B200CONST_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define B200C_API __attribute__((visibility("default")))
#else
#define B200C_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define B200C_MAX_RANK 8

/* ---- element types ------------------------------------------------------
 * dtype = (class << 8) | bit width.  Integer signedness follows MLIR:
 * signless (i8), signed (si8), unsigned (ui8).  The reference treats signless
 * integers as unsigned when it reads values
 * (src/vpux_compiler/include/vpux/compiler/dialect/const/utils/content.hpp:253-299).
 */
#define B200C_CLS_FLOAT 1
#define B200C_CLS_BFLOAT 2
#define B200C_CLS_INT 3  /* signless */
#define B200C_CLS_SINT 4 /* signed   */
#define B200C_CLS_UINT 5 /* unsigned */
#define B200C_DTYPE(cls, bits) (((cls) << 8) | (bits))
#define B200C_DTYPE_BITS(dt) ((dt)&0xFF)
#define B200C_DTYPE_CLASS(dt) (((dt) >> 8) & 0xFF)

#define B200C_F64 B200C_DTYPE(B200C_CLS_FLOAT, 64)
#define B200C_F32 B200C_DTYPE(B200C_CLS_FLOAT, 32)
#define B200C_F16 B200C_DTYPE(B200C_CLS_FLOAT, 16)
#define B200C_BF16 B200C_DTYPE(B200C_CLS_BFLOAT, 16)
#define B200C_I1 B200C_DTYPE(B200C_CLS_INT, 1)
#define B200C_UI1 B200C_DTYPE(B200C_CLS_UINT, 1)
#define B200C_I4 B200C_DTYPE(B200C_CLS_INT, 4)
#define B200C_SI4 B200C_DTYPE(B200C_CLS_SINT, 4)
#define B200C_UI4 B200C_DTYPE(B200C_CLS_UINT, 4)
#define B200C_I8 B200C_DTYPE(B200C_CLS_INT, 8)
#define B200C_SI8 B200C_DTYPE(B200C_CLS_SINT, 8)
#define B200C_UI8 B200C_DTYPE(B200C_CLS_UINT, 8)
#define B200C_I16 B200C_DTYPE(B200C_CLS_INT, 16)
#define B200C_SI16 B200C_DTYPE(B200C_CLS_SINT, 16)
#define B200C_UI16 B200C_DTYPE(B200C_CLS_UINT, 16)
#define B200C_I32 B200C_DTYPE(B200C_CLS_INT, 32)
#define B200C_SI32 B200C_DTYPE(B200C_CLS_SINT, 32)
#define B200C_UI32 B200C_DTYPE(B200C_CLS_UINT, 32)
#define B200C_I64 B200C_DTYPE(B200C_CLS_INT, 64)
#define B200C_SI64 B200C_DTYPE(B200C_CLS_SINT, 64)
#define B200C_UI64 B200C_DTYPE(B200C_CLS_UINT, 64)

/* ---- quantisation kinds (mlir::quant::UniformQuantized[PerAxis]Type) ---- */
#define B200C_Q_NONE 0
#define B200C_Q_PER_TENSOR 1
#define B200C_Q_PER_AXIS 2

/*
 * Tensor type: what vpux::NDTypeInterface carries for a constant
 * (shape, element type, DimsOrder).  For a quantised element type `dtype` is
 * the normalised storage integer (si8/ui8/si4/ui4,
 * src/vpux_compiler/src/utils/quantization.cpp:47-54) and the q* fields hold
 * the quantisation parameters.  `scales`/`zps` are borrowed, `nq` entries each
 * (1 for per-tensor).  `order[k]` is the logical dimension stored at memory
 * position k, k = 0 being the outermost (DimsOrder::toPermutation); NHWC is
 * {0,2,3,1}.
 */
typedef struct b200c_type {
    int32_t dtype;
    int32_t rank;
    int64_t shape[B200C_MAX_RANK];
    uint8_t order[B200C_MAX_RANK];
    int32_t qkind;
    int32_t qaxis;
    int32_t qexpressed; /* dtype of the expressed type (f32/f16) */
    int32_t _pad;
    int64_t qmin, qmax; /* storageTypeMin / storageTypeMax */
    int64_t nq;
    const double* scales;
    const int64_t* zps;
} b200c_type;

/* ---- transformation kinds: one per reference attribute mnemonic ----------
 * (src/vpux_compiler/tblgen/vpux/compiler/dialect/const/attributes.td)       */
enum b200c_xform_kind {
    B200C_X_CONVERT_ELEM_TYPE = 1, /* type.dtype (+quant none)                 */
    B200C_X_QUANT_CAST = 2,        /* type.q*; type.dtype == 0 -> strip quant   */
    B200C_X_DEQUANTIZE = 3,
    B200C_X_RESCALE = 4,      /* f = scale                                       */
    B200C_X_ADD = 5,          /* f = bias                                        */
    B200C_X_REORDER = 6,      /* a[0..rank) = new order permutation              */
    B200C_X_SUBVIEW = 7,      /* a = offset, b = shape                           */
    B200C_X_PAD_WITH_ZERO = 8, /* a = padBefore, b = padAfter                    */
    B200C_X_BIT_PACK = 9,     /* i0 = width (4)                                  */
    B200C_X_GET_SPARSITY_MAP = 10,
    B200C_X_SPARSIFY = 11,    /* i0 = compressOutputType, aux = numActualElements */
    B200C_X_SWIZZLE_CONSTANT = 12, /* i0 = swizzle key, i1 = arch (3 = VPUX37XX)  */
    B200C_X_RESHAPE = 13,     /* b = new shape, n = new rank                     */
    B200C_X_CHANGE_SHAPE_AND_ELEM_TYPE = 14, /* b = shape, type = element type   */
    B200C_X_BROADCAST = 15,   /* i0 = axis, i1 = value                           */
    B200C_X_TRANSPOSE = 16,   /* a = order permutation                           */
    B200C_X_REVERSE = 17,     /* i0 = axis                                       */
    B200C_X_EXPAND_DILATED = 18, /* a[0..1] = dilations                          */
    /* relocate_weights_table.cpp:122-203.  n = clusters, a[k] = offsets[k] (first output channel of
     * cluster k), b[k] = weightsPtr[k], i0 = sparsityPtr, i1 = weightsElemBitSize (0 = absent),
     * aux = numElems of the weights compression scheme (one per output channel; NULL = no
     * compression), f = its alignment in bytes (0 = the default 16).                              */
    B200C_X_RELOCATE_WEIGHTS_TABLE = 19,
    /* Synthetic producer step with no reference counterpart: per-channel
     * (axis 0) quantisation of a float tensor.  i0 = scheme:
     *   0: symmetric int8  scale = max|w|/127, zp = 0, round-half-even, clamp [-127,127]
     *   1: asymmetric u4   scale = (max-min)/15, zp = clamp(rint(-min/scale),0,15)
     * side0 / side1 receive the per-channel f32 scales / i32 zero points
     * (same residency as the fold output).  The result holds the integral
     * values in f32 storage; follow it with ConvertElemType + QuantCast.      */
    B200C_X_QUANTIZE_SYNTH = 100
};

#define B200C_QSYNTH_SYM_I8 0
#define B200C_QSYNTH_ASYM_U4 1

typedef struct b200c_xform {
    int32_t kind;
    int32_t n;                  /* entries used in a[] / b[]                    */
    int64_t a[B200C_MAX_RANK];
    int64_t b[B200C_MAX_RANK];
    double f;
    int64_t i0, i1;
    b200c_type type;
    const int64_t* aux;
    int64_t naux;
    void* side0;
    void* side1;
} b200c_xform;

/* ---- return codes --------------------------------------------------------- */
#define B200C_OK 0
#define B200C_NOT_SMALLER 1       /* compress: the reference's mlir::failure()   */
#define B200C_ERR_INVALID (-1)    /* malformed descriptor / argument             */
#define B200C_ERR_THROW (-2)      /* the reference would VPUX_THROW here         */
#define B200C_ERR_CUDA (-3)       /* CUDA runtime failure or no device           */
#define B200C_ERR_NOMEM (-4)      /* device or host allocation failed            */
#define B200C_ERR_CAPACITY (-5)   /* output buffer too small                     */
#define B200C_ERR_UNSUPPORTED (-6) /* valid in the reference, not built here     */

/* ---- context ----------------------------------------------------------------
 * One context per (host thread, device).  It owns a CUDA stream, a growing
 * scratch arena and pinned staging memory.  Calls on different contexts may
 * run concurrently (the reference folds from many threads at once:
 * src/vpux_compiler/src/dialect/VPUIP/graph-schema/export.cpp:465 and
 * src/vpux_compiler/src/dialect/const/utils/constant_folding_in_background.cpp:57-100);
 * calls on one context are serialised by an internal mutex.                   */
typedef struct b200c_ctx b200c_ctx;
B200C_API int b200c_create(int device, b200c_ctx** out);
B200C_API void b200c_destroy(b200c_ctx* ctx);
/* Device memory for the library's own scratch.  The reference allocates every intermediate
 * buffer of a fold on the host heap (Const::Content::allocTempBuffer,
 * src/vpux_compiler/src/dialect/const/utils/content.cpp:32-47); here intermediates, staged inputs
 * and launch tables live in a per-context arena of device blocks (64 MiB or more each, kept and
 * reused across calls).  By default the blocks come from cudaMalloc; a host that runs its own
 * device memory pool installs its allocator here.  alloc_fn returns a device pointer aligned to
 * 256 bytes, or NULL when it has no memory -- the call in progress then fails with
 * B200C_ERR_NOMEM and the context stays usable.  Both functions may be called from the
 * library's planning threads, concurrently.  Installing (or removing, with two NULLs) an
 * allocator waits for the context's stream and returns every block to the allocator it came
 * from.  b200c_dev_alloc is not affected.                                      */
typedef void* (*b200c_alloc_fn)(void* user, size_t bytes);
typedef void (*b200c_free_fn)(void* user, void* ptr);
B200C_API int b200c_set_allocator(b200c_ctx* ctx, b200c_alloc_fn alloc_fn, b200c_free_fn free_fn, void* user);
/* Use `stream` (a cudaStream_t) for all later work of this context; NULL
 * restores the context's own stream.                                          */
B200C_API int b200c_set_stream(b200c_ctx* ctx, void* stream);
B200C_API void* b200c_get_stream(b200c_ctx* ctx);
/* Waits for the context's stream (and its transfer stream, if used) and reports device-side errors. */
B200C_API int b200c_synchronize(b200c_ctx* ctx);
/* Number of kernels of this library launched through the context so far.     */
B200C_API int64_t b200c_launch_count(b200c_ctx* ctx);
/* Thread-local message of the last failing call on this thread.              */
B200C_API const char* b200c_last_error(void);
B200C_API const char* b200c_version(void);

/* ---- type inference -----------------------------------------------------------
 * Const::ContentAttr::inferFinalType
 * (src/vpux_compiler/src/dialect/const/attributes/content.cpp:373-381) and each
 * attribute's inferOutputType.  `out->scales` / `out->zps` must point to
 * caller storage of `out->nq` entries on entry when the result can be
 * per-axis quantised; on return nq is the count written.  Pure host code.     */
B200C_API int b200c_infer_type(const b200c_type* in, const b200c_xform* chain, int n, b200c_type* out);

/* Index at which ContentAttr::addTransformation inserts a new transformation
 * (getInsertionPosition, content.cpp:268-299): NONE before PREFERRED_LAST before
 * LAST; a second LAST is an error.  `kinds` are the b200c_xform_kind values of
 * the existing list.                                                          */
B200C_API int b200c_insert_position(const int32_t* kinds, int n, int32_t new_kind, int* pos);

/* Byte size of a tensor of this type: NDTypeInterface::getTotalAllocSize
 * (src/vpux_compiler/src/core/type_interfaces.cpp:148-162).                   */
B200C_API int64_t b200c_total_alloc_size(const b200c_type* t);

/* ---- folding -------------------------------------------------------------------
 * Const::ContentAttr::fold() followed by Const::Content::copyTo()
 * (content.cpp:167-193, src/vpux_compiler/src/dialect/const/utils/content.cpp:184-207),
 * i.e. what Const::DeclareOp::getContent() + copyTo hands to the constant-folding
 * pass (src/vpux_compiler/src/dialect/const/passes/constant_folding.cpp:27-77),
 * the blob writer (export.cpp:465-479) and the compression pass.
 *
 *  base/data/nbytes : the base ElementsAttr: type and raw bytes; `is_splat`
 *                     means `data` holds a single element.
 *  data_on_device   : `data` is a device pointer on the context's device.
 *  out/out_cap      : destination; `out_on_device` as above.  The bytes are
 *                     exactly those copyTo writes; *out_bytes is their count.
 *                     Bytes of `out` beyond *out_bytes are not touched.
 *  out_type         : type of the folded Content (may be NULL); pointer rules
 *                     as for b200c_infer_type.
 * The call returns after the result is complete (it synchronises the
 * context's stream) unless out_on_device != 0 and B200C_FOLD_ASYNC is set in
 * `flags`, in which case data-dependent errors are reported by the next
 * synchronising call on the context.                                          */
#define B200C_FOLD_ASYNC 1
B200C_API int b200c_fold(b200c_ctx* ctx, const b200c_type* base, const void* data, size_t nbytes, int is_splat,
               int data_on_device, const b200c_xform* chain, int n, void* out, size_t out_cap, int out_on_device,
               size_t* out_bytes, b200c_type* out_type, int flags);

/* Many constants in one call: the whole-model form of b200c_fold, standing where the reference
 * loops over every Const::DeclareOp of a model (serializeBinaryData,
 * src/vpux_compiler/src/dialect/VPUIP/graph-schema/export.cpp:465-479).  Items are independent;
 * kernels of the same kind are issued as one launch over all items, so small constants do not pay
 * one launch each.  data_on_device / out_on_device / flags apply to every item; out_bytes of each
 * item receives the bytes written.  Side outputs of QuantizeSynth are written in place when the
 * outputs are on the device.  Planning (type inference, view composition, launch parameters) of
 * large batches runs on a small pool of host threads (B200C_PLAN_THREADS overrides their number,
 * 0 or 1 = none), as the reference folds constants in a parallel loop; all launches still go to the
 * context's one stream.  When an item's size depends on its data (Sparsify without
 * numActualElements) the call waits for the device once, at its end, even with B200C_FOLD_ASYNC. */
typedef struct b200c_fold_item {
    const b200c_type* base;
    const void* data;
    size_t nbytes;
    int32_t is_splat;
    int32_t n; /* transformations in chain */
    const b200c_xform* chain;
    void* out;
    size_t out_cap;
    size_t out_bytes; /* result */
} b200c_fold_item;
B200C_API int b200c_fold_batch(b200c_ctx* ctx, b200c_fold_item* items, int count, int data_on_device, int out_on_device,
                               int flags);

/* Per-output-channel count of elements that differ from the sparsify value:
 * vpux::countNonSparseElementsPerOC (src/vpux_compiler/src/utils/sparsity.cpp:28-72)
 * applied to the folded content of (base, chain).  counts: host int64[shape[0]].  */
B200C_API int b200c_count_nonsparse_per_oc(b200c_ctx* ctx, const b200c_type* base, const void* data, size_t nbytes,
                                 int is_splat, int data_on_device, const b200c_xform* chain, int n,
                                 int64_t* counts, int64_t ncounts);

/* ---- weight compression ----------------------------------------------------------
 * Stands where vpux::BitCompactorCodec::compress calls
 * btc27::BitCompactor::{GetCompressedSizeBound, CompressArray}
 * (src/vpux_compiler/src/utils/bit_compactor_codec.cpp:15-42).  The bitstream is
 * this library's own block format (64-byte blocks, per-block mode selection),
 * not BitCompactor's: the BitCompactor sources are not part of the reference
 * tree.  b200c_btc_compress returns B200C_NOT_SMALLER when the stream would not
 * be smaller than the input, as the reference's codec returns failure.        */
B200C_API int b200c_btc_bound(size_t n, size_t* bound);
B200C_API int b200c_btc_compress(b200c_ctx* ctx, const void* in, size_t n, int in_on_device, void* out, size_t cap,
                       int out_on_device, size_t* out_n);
B200C_API int b200c_btc_decompress(b200c_ctx* ctx, const void* in, size_t n, int in_on_device, void* out, size_t cap,
                         int out_on_device, size_t* out_n);

/* Allocation-free form of b200c_btc_compress (no counterpart in the reference).
 *
 * For callers that cannot let this library allocate GPU memory: a process whose device memory is
 * claimed in full by its own pool, so that one more cudaMalloc fails or eats into that pool, or one
 * that cannot afford the device-wide synchronisation an allocation brings while other streams run.
 * This call allocates nothing, on the device or through any library: `in` and `out` are the
 * caller's device buffers and the working arrays come from a fixed buffer inside the library
 * image (about 1 MiB, held by every GPU that loads the library until the process exits).
 *
 *  - n may be at most B200C_NOALLOC_MAX_INPUT bytes (16 MiB); larger inputs are refused with
 *    B200C_ERR_CAPACITY and a message saying so.  cap must be at least b200c_btc_bound(n).
 *  - `device` is the CUDA device of in/out, `stream` a cudaStream_t on it (NULL: the default
 *    stream).  The call blocks until the stream has finished the work and reads the result size
 *    back, so it must never be made while `stream` is being captured.  The calling thread's current
 *    device is the same after the call as before it.
 *  - The first call on a device also looks up the address of the fixed buffer (once per device).
 *  - All calls on one device share the fixed buffer.  Each call rewrites what it reads, so calls
 *    may follow one another freely, but two calls whose GPU work overlaps (two threads, two
 *    streams) race on it: serialise them.
 * Output and return codes are those of b200c_btc_compress (B200C_NOT_SMALLER included).          */
#define B200C_NOALLOC_MAX_INPUT ((size_t)16 << 20)
B200C_API int b200c_btc_compress_noalloc(int device, const void* in_dev, size_t n, void* out_dev, size_t cap,
                                         void* stream, size_t* out_n);

/* Batched form used for whole-model folding: `count` independent buffers that
 * already reside on the device are compressed with one analysis launch, one
 * device prefix sum and one emit launch.  sizes/offsets are host arrays;
 * out_sizes[i] receives the stream length of buffer i (B200C_NOT_SMALLER cases
 * are reported through not_smaller[i] = 1 and store the input unchanged).     */
B200C_API int b200c_btc_compress_batch(b200c_ctx* ctx, int count, const void* const* in_dev, const size_t* sizes,
                             void* out_dev, size_t out_cap, size_t* out_offsets, size_t* out_sizes,
                             int32_t* not_smaller);

/* In-place form of the batched compression, for blob writers that fold every constant straight
 * into its slot of the blob: a buffer whose stream is smaller than the buffer gets the stream
 * written over its own first bytes (out_sizes[i] = stream length, compressed[i] = 1); a buffer that
 * would not shrink is left untouched (out_sizes[i] = sizes[i], compressed[i] = 0) and costs one read
 * of its bytes and no write at all.  This is the outcome of the reference's compression pass --
 * replace the constant only "if smaller" (compress_weights_btc.cpp:130-136) -- without moving
 * incompressible constants.  Buffers are device memory; the call synchronises.                    */
B200C_API int b200c_btc_compress_inplace_batch(b200c_ctx* ctx, int count, void* const* bufs_dev, const size_t* sizes,
                                               size_t* out_sizes, int32_t* compressed);

/* The same in two steps, for writers that fold the next group of constants while the device still
 * compresses the previous one: _begin queues the work on the context's stream and returns a
 * ticket at once; _end waits for that work only (not for anything queued after it) and hands
 * the sizes back as b200c_btc_compress_inplace_batch does.  The buffers must not be touched by
 * the caller between the two calls.  Up to 8 tickets may be open per context.  A device-side
 * error of earlier work (the sticky error word) is reported by the next call that waits for the
 * whole stream, e.g. b200c_synchronize.                                                           */
B200C_API int b200c_btc_compress_inplace_begin(b200c_ctx* ctx, int count, void* const* bufs_dev, const size_t* sizes,
                                               int* ticket);
B200C_API int b200c_btc_compress_inplace_end(b200c_ctx* ctx, int ticket, size_t* out_sizes, int32_t* compressed);

/* ---- splat detection -------------------------------------------------------------
 * "All elements equal" test of a raw buffer: detectSplatElementWise, which the reference runs when
 * it wraps a dense resource (src/vpux_compiler/src/dialect/const/attributes/content.cpp:103-137,
 * called from wrapBaseContent :143-159) -- there a memcmp loop over the elements, here one
 * reduction kernel.  elem_bytes is 1, 2, 4 or 8.  *is_splat = 1 when every element equals the
 * first (a single element is a splat; an empty buffer is not, as in detectSplatManually).  Errors
 * as the reference throws them: fewer bytes than one element, or a length that is not a multiple
 * of the element size.  A caller passes the answer on as `is_splat` of b200c_fold together with
 * nbytes = elem_bytes.                                                                          */
B200C_API int b200c_detect_splat(b200c_ctx* ctx, const void* data, size_t nbytes, int elem_bytes, int data_on_device,
                                 int* is_splat);

/* ---- multi-GPU exchange --------------------------------------------------------------
 * The reference writes every constant of a model into one blob from a parallel loop in one
 * process (serializeBinaryData, src/vpux_compiler/src/dialect/VPUIP/graph-schema/export.cpp:465-479).
 * When the constants are sharded over the GPUs of one machine, one process per GPU, these calls
 * carry the finished slots into the blob buffer of the assembling rank over NVLink.  They have no
 * further counterpart in the reference (which is a single process).
 *
 * b200c_ipc_export describes a range of a b200c_dev_alloc allocation so that another process on
 * the same machine can map it with b200c_ipc_open (CUDA IPC; peer access is enabled on demand);
 * the returned pointer is valid in device code and in the copy calls below.
 *
 * b200c_copy_segments_async queues `count` copies src -> dst on the context's transfer stream,
 * ordered after everything queued on the context's stream so far; it returns at once.  dst may
 * be a mapped peer range (push over NVLink) or pinned host memory (download).
 *   wait_flag/wait_value : if not NULL, a device word of this GPU; the copies start only when it
 *                          holds at least wait_value (the assembling rank's release of its buffer);
 *   done_flag/done_value : if not NULL, a device word (usually in the peer's memory) that
 *                          receives done_value after all bytes have landed;
 *   mode 0               : a copy kernel with plain 128-bit loads and stores (`ctas` CTAs; peer
 *                          memory is only ever stored to); a wait that times out cancels the copy;
 *   mode 1               : the copy engine (one cudaMemcpyAsync per segment);
 *   mode 2               : a copy kernel built on the SM's bulk-copy unit (cp.async.bulk through a
 *                          shared-memory ring, no multicast): the form for a pusher whose SMs
 *                          fold the next chunk meanwhile, since stalled NVLink stores then queue
 *                          in the copy unit instead of the load/store pipeline.  Same cancel rule
 *                          as mode 0; a copy that stalls inside the kernel sets bit 2 of the status.
 * b200c_wait_flags queues, on the context's stream (or, with on_transfer_stream != 0, on its
 * transfer stream, so that only the copies queued there afterwards are held back), a bounded wait
 * until each of `count` consecutive device words holds at least `value`; b200c_signal_flags queues
 * stores of `value`
 * to the given device words (peer memory allowed).  No wait spins for more than timeout_ms:
 * it then records the failure and lets the stream continue.  b200c_exchange_status waits for
 * both streams and returns the failures since the last call in *timed_out (bit 0: a release
 * wait of a pusher, bit 1: a done wait of the assembling rank, bit 2: a stalled bulk copy) -- the caller turns a non-zero
 * value into its own error.                                                                      */
typedef struct b200c_ipc_handle {
    unsigned char handle[64];
    uint64_t offset; /* of the exported address inside the allocation */
    uint64_t size;
} b200c_ipc_handle;
typedef struct b200c_copy_seg {
    const void* src;
    void* dst;
    size_t n;
} b200c_copy_seg;
B200C_API int b200c_ipc_export(b200c_ctx* ctx, void* dev_ptr, size_t size, b200c_ipc_handle* out);
B200C_API int b200c_ipc_open(b200c_ctx* ctx, const b200c_ipc_handle* h, void** mapped);
B200C_API int b200c_ipc_close(b200c_ctx* ctx, void* mapped);
B200C_API int b200c_copy_segments_async(b200c_ctx* ctx, const b200c_copy_seg* segs, int count, const uint64_t* wait_flag,
                                        uint64_t wait_value, uint64_t* done_flag, uint64_t done_value,
                                        unsigned timeout_ms, int mode, int ctas);
/* The same copies, ordered after the work of a compression ticket (b200c_btc_compress_inplace_begin;
 * the ticket may have been collected already, as long as no later _begin has reused it) instead
 * of after everything queued on the context's stream: a chunk travels as soon as it is complete
 * although the next chunk's kernels are queued behind it.                                          */
B200C_API int b200c_copy_segments_after(b200c_ctx* ctx, int ticket, const b200c_copy_seg* segs, int count,
                                        const uint64_t* wait_flag, uint64_t wait_value, uint64_t* done_flag,
                                        uint64_t done_value, unsigned timeout_ms, int mode, int ctas);
B200C_API int b200c_wait_flags(b200c_ctx* ctx, const uint64_t* flags_dev, int count, uint64_t value, unsigned timeout_ms,
                               int on_transfer_stream);
B200C_API int b200c_signal_flags(b200c_ctx* ctx, uint64_t* const* targets, int count, uint64_t value);
B200C_API int b200c_exchange_status(b200c_ctx* ctx, int* timed_out);
/* Makes the context's stream wait (on the device, without blocking the host) for everything queued
 * on its transfer stream so far: a pusher calls it before it overwrites slots it has pushed, the
 * assembling rank before it releases a buffer whose download is still queued.                      */
B200C_API int b200c_stream_join(b200c_ctx* ctx);

/* ---- buffer digest -------------------------------------------------------------------
 * 64-bit digest of each of `count` device buffers (no counterpart in the reference; a
 * measurement aid): used to show that the blob assembled from N GPUs holds the same bytes per
 * constant as the one folded on a single GPU, without moving gigabytes to the host.
 *   digest(bytes, n) = mix(0x9E3779B97F4A7C15 * (n + 1) + sum_j mix(word_j ^ (0xD6E8FEB86659FD93 * (j + 1))))
 * over the little-endian 64-bit words of the buffer (the last one zero-extended), modulo 2^64,
 * mix = the splitmix64 finaliser.  out: host array; the call synchronises.                       */
B200C_API int b200c_digest64_batch(b200c_ctx* ctx, int count, const void* const* bufs_dev, const size_t* sizes,
                                   uint64_t* out);

/* ---- synthetic weights ----------------------------------------------------------
 * Counter-based seeded generator (Philox-4x32-10 keyed by seed and stream)
 * used by the benchmark so that inputs never cross PCIe (no counterpart in the
 * reference; the benchmark configurations only name distributions and a seed).
 * dist: 0 = normal (p0 = sigma, Box-Muller), 1 = uniform int8 in [-127,127] with
 * Bernoulli(p0) zeros, 2 = discretised Laplace(0, p0) clipped to [-127,127] with a
 * fraction p1 of exact zeros.  dtype: B200C_F32, B200C_F16 or B200C_SI8.  Element i
 * depends only on (seed, stream_id, i).  The logarithm, sine and cosine are fixed
 * polynomial evaluations in IEEE single precision (no math library), so a CPU
 * restatement produces the same bytes.                                        */
B200C_API int b200c_synth_fill(b200c_ctx* ctx, void* dst_dev, int64_t count, int32_t dtype, int32_t dist, double p0,
                     double p1, uint64_t seed, uint64_t stream_id);

/* ---- device memory helpers (so that callers need no CUDA runtime of their own) */
B200C_API int b200c_dev_alloc(b200c_ctx* ctx, size_t n, void** out);
B200C_API int b200c_dev_free(b200c_ctx* ctx, void* p);
B200C_API int b200c_host_alloc_pinned(size_t n, void** out);
B200C_API int b200c_host_free_pinned(void* p);
B200C_API int b200c_dev_memset(b200c_ctx* ctx, void* dst_dev, int value, size_t n); /* queued on the context's stream */
B200C_API int b200c_memcpy_h2d(b200c_ctx* ctx, void* dst_dev, const void* src, size_t n);
B200C_API int b200c_memcpy_d2h(b200c_ctx* ctx, void* dst, const void* src_dev, size_t n);

#ifdef __cplusplus
}
#endif
#endif /* B200CONST_H_ */
