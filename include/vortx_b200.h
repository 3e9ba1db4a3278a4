/*
 * vortx_b200 — C ABI of the B200 (sm_100a) matmul path for vortx.
 *
 * This is the boundary a vortx build binds instead of khal for GEMM, GEMV and the
 * device-buffer plumbing around them.  Plain pointers and sizes only; every function
 * returns a vx_status and never throws or aborts.  A context owns one CUDA stream and
 * all work it is given is ordered on that stream and asynchronous until
 * vx_synchronize / vx_download.  A context is not thread-safe; distinct contexts (one
 * per GPU) may be driven from distinct threads.
 *
 * Each declaration names the reference interface it stands in for, by file:line in
 * the vortx source tree (v0.3.0).
 */
#ifndef VORTX_B200_H
#define VORTX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define VX_API
#else
#define VX_API __attribute__((visibility("default")))
#endif

typedef int32_t vx_status;
enum {
    VX_OK = 0,
    VX_ERR_INVALID_ARGUMENT = 1, /* null pointer, zero/odd size, unknown enum value          */
    VX_ERR_SHAPE = 2,            /* the shape checks of src/linalg/gemm.rs:70-104 failed      */
    VX_ERR_OUT_OF_BOUNDS = 3,    /* a layout addresses elements beyond the stated capacity    */
    VX_ERR_CUDA = 4,             /* a CUDA runtime / driver call failed (see vx_last_error)   */
    VX_ERR_OUT_OF_MEMORY = 5,    /* cudaMalloc failed                                         */
    VX_ERR_UNSUPPORTED = 6,      /* the requested kernel cannot take these operands           */
    VX_ERR_DEVICE_TIMEOUT = 7,   /* a bounded device-side wait gave up; results are invalid   */
    VX_ERR_NO_DEVICE = 8,        /* no usable sm_100 device / driver                          */
    VX_ERR_COLLECTIVE = 9        /* an NCCL call failed, or NCCL could not be loaded          */
};

/* Thread-local text of the last failure on this thread ("" if none). */
VX_API const char* vx_last_error(void);
VX_API const char* vx_version(void);

/* ------------------------------------------------------------------ context ---- */
/* Replaces khal's GpuBackend::Cuda(Cuda::new(ordinal)) — src/linalg/gemm.rs:353.   */
typedef struct vx_context vx_context;

VX_API vx_status vx_context_create(int32_t device, vx_context** out);
/* Same, but work is ordered on a stream the caller owns (a cudaStream_t). */
VX_API vx_status vx_context_create_on_stream(int32_t device, void* cuda_stream, vx_context** out);
VX_API vx_status vx_context_destroy(vx_context* ctx);
/* backend.synchronize() — src/linalg/gemm.rs:421, examples/gemm_bench.rs:77. */
VX_API vx_status vx_synchronize(vx_context* ctx);
VX_API vx_status vx_context_device(const vx_context* ctx, int32_t* device);
VX_API vx_status vx_context_stream(const vx_context* ctx, void** cuda_stream);
/* Number of kernels this context has launched since creation (copies excluded). */
VX_API vx_status vx_context_launch_count(const vx_context* ctx, uint64_t* count);

/* ------------------------------------------------------------------- memory ---- */
/* backend.uninit_buffer(len, usage) — src/tensor/tensor_impl.rs:69.  cudaMalloc. */
VX_API vx_status vx_alloc(vx_context* ctx, size_t bytes, void** device_ptr);
VX_API vx_status vx_free(vx_context* ctx, void* device_ptr);
/* backend.init_buffer(data, usage) / write_buffer(buf, offset, data) —
 * src/tensor/tensor_impl.rs:105, :715; src/shapes.rs:581, :603.  Stream-ordered H2D. */
VX_API vx_status vx_upload(vx_context* ctx, void* device_dst, const void* host_src, size_t bytes);
/* backend.slow_read_buffer(buf, host) — src/linalg/gemm.rs:423-426.  Blocks until done. */
VX_API vx_status vx_download(vx_context* ctx, void* host_dst, const void* device_src, size_t bytes);
/* slow_read_buffer of a strided view (src/tensor/tensor_ref.rs:101-103 carries the offset, the layout the
 * row stride): `rows` pieces of `width_bytes`, src_pitch bytes apart on the device, land dst_pitch bytes
 * apart on the host, in one copy.  Blocks until done. */
VX_API vx_status vx_download_2d(vx_context* ctx, void* host_dst, size_t dst_pitch, const void* device_src,
                                size_t src_pitch, size_t width_bytes, size_t rows);
/* encoder.copy_buffer_to_buffer(src, src_off, dst, dst_off, len) —
 * src/tensor/tensor_impl.rs:207-213.  Offsets are applied by the caller. */
VX_API vx_status vx_copy(vx_context* ctx, void* device_dst, const void* device_src, size_t bytes);
VX_API vx_status vx_memset(vx_context* ctx, void* device_dst, int value, size_t bytes);
/* Page-locked host staging memory for uploads/downloads that should overlap. */
VX_API vx_status vx_host_alloc(size_t bytes, void** host_ptr);
VX_API vx_status vx_host_free(void* host_ptr);

/* -------------------------------------------------------------------- shapes ---- */
/* vortx-shaders/src/linalg/shape.rs:9-29 — the kernel-side shape, eight u32 in
 * elements: sizes n,c,h,w (h = rows, w = columns) then the four strides. */
typedef struct {
    uint32_t n, c, h, w;
    uint32_t n_stride, c_stride, h_stride, w_stride;
} vx_shape;

/* vortx-shaders/src/linalg/shape.rs:112-123 — passed by value, as push constants were
 * meant to be; there is no uniform-buffer cache (src/shapes.rs:541-640 goes away). */
typedef struct {
    vx_shape out, lhs, rhs;
} vx_shapes3;

/* --------------------------------------------------------------------- GEMM ---- */
typedef enum {
    VX_GEMM_AUTO = 0,       /* Gemm::dispatch's rule — src/linalg/gemm.rs:111-118: the exact SIMT
                               kernel; tiled when M >= 32 || N >= 32, else one thread per element */
    VX_GEMM_NAIVE = 1,      /* gemm_naive — vortx-shaders/src/linalg/gemm.rs:197-237              */
    VX_GEMM_SIMT_EXACT = 2, /* gemm_tiled — vortx-shaders/src/linalg/gemm.rs:41-194, bit for bit   */
    VX_GEMM_TF32 = 3        /* tcgen05 tensor-core kernel, TF32 inputs, f32 accumulate; operands
                               that TMA cannot address fall back to SIMT_EXACT                     */
} vx_gemm_mode;

/* The `.call(pass, grid, shapes.., out, lhs, rhs)` level — src/linalg/gemm.rs:131-151,
 * :217-226, :276-285.  out = lhs * rhs for every (n, c) matrix pair; out is overwritten.
 * Pointers are device pointers already advanced by the view offset
 * (src/tensor/tensor_ref.rs:101-103).  cap_* are the element counts reachable from each
 * pointer; a shape that reaches beyond them is refused with VX_ERR_OUT_OF_BOUNDS (pass 0
 * to skip the check).  No shape-compatibility check is made at this level, as
 * dispatch_naive / dispatch_tiled make none. */
VX_API vx_status vx_gemm_f32(vx_context* ctx, vx_gemm_mode mode, float* out, const float* lhs,
                             const float* rhs, const vx_shapes3* shapes, uint64_t cap_out,
                             uint64_t cap_lhs, uint64_t cap_rhs);
/* Which kernel the last vx_gemm_f32 on this context ran: 1 naive, 2 SIMT tiled (vector
 * loads), 3 tcgen05 TF32, 4 SIMT tiled (generic strides). */
VX_API vx_status vx_gemm_last_kernel(const vx_context* ctx, int32_t* kernel);

/* ------------------------------------------------- block-quantised weights ---- */
/* No reference counterpart: vortx has no quantised type.  Entry points follow the
 * shape of its matrix-times-[K,1] use of Gemm::dispatch (src/linalg/gemm.rs:46, :373-387).
 *
 * Host block streams (what a caller holds): rows*cols/32 blocks, row after row.
 *   Q8_0 block, 34 B: f16 d | int8 q[32]                 w[i]    = d * q[i]
 *   Q4_0 block, 18 B: f16 d | u8 qs[16]                  w[i]    = d * ((qs[i] & 15) - 8)
 *                                                        w[i+16] = d * ((qs[i] >> 4) - 8)
 * Device form (vx_qweights): the same bytes split into a plane of quants (16-byte
 * aligned rows) and a plane of scales, so every load is a full aligned vector. */
typedef enum { VX_Q8_0 = 0, VX_Q4_0 = 1 } vx_qtype;
typedef struct vx_qweights vx_qweights;

VX_API size_t vx_qblock_bytes(vx_qtype t);
/* Host quantisers.  cols % 32 == 0.  blocks receives rows*cols/32 * vx_qblock_bytes(t). */
VX_API vx_status vx_quantize(vx_qtype t, const float* w, size_t rows, size_t cols, void* blocks);
VX_API vx_status vx_dequantize_host(vx_qtype t, const void* blocks, size_t rows, size_t cols,
                                    float* w);
/* Upload a host block stream; rows x cols logical weights. */
VX_API vx_status vx_qweights_upload(vx_context* ctx, vx_qtype t, const void* blocks, size_t rows,
                                    size_t cols, vx_qweights** out);
/* The same weights quantised ON the device from an f32 matrix that is already there (rows row_stride
 * elements apart), straight into the planar layout: no host pass, no upload.  Bit-identical to
 * vx_quantize + vx_qweights_upload of the same values.  Stream-ordered. */
VX_API vx_status vx_qweights_from_device(vx_context* ctx, vx_qtype t, const float* w_device, size_t rows,
                                         size_t cols, size_t row_stride, vx_qweights** out);
VX_API vx_status vx_qweights_free(vx_context* ctx, vx_qweights* w);
VX_API vx_status vx_qweights_info(const vx_qweights* w, int32_t* qtype, size_t* rows, size_t* cols,
                                  size_t* device_bytes);
/* Device dequantisation into a row-major f32 matrix (rows*cols floats). */
VX_API vx_status vx_dequantize(vx_context* ctx, const vx_qweights* w, float* device_out);
/* y[v*y_stride + r] = sum_c W[r, c] * x[v*x_stride + c], v < batch.
 * x and y are device pointers; strides in elements between batch vectors.
 * Arithmetic of the default kernel: each 16-byte chunk of a row (32 Q4_0 / 16 Q8_0 weights) is multiplied
 * with x held as 24-bit fixed point relative to the largest |x| of that chunk; the integer sum of a chunk
 * is exact, and the chunk sums, scaled by d * sx, are accumulated in f32.  An x value therefore carries an
 * absolute error of up to 2^-24 of its chunk's largest value: the same as f32 for values near the chunk's
 * maximum, coarser for values far below it (a 1e-3 next to a 1e4 keeps about 1 significant bit; an f32
 * accumulation would lose the same value in the rounding of the sum).  A NaN or infinity in x makes every
 * row NaN.  The result is within 1e-4 (max-norm relative) of the f64 product at the sizes tested. */
VX_API vx_status vx_gemv_q(vx_context* ctx, const vx_qweights* w, const float* x, size_t x_stride,
                           float* y, size_t y_stride, size_t batch);
/* Same, for a contiguous slab of rows [row0, row0+nrows): y receives nrows values per vector. */
VX_API vx_status vx_gemv_q_rows(vx_context* ctx, const vx_qweights* w, size_t row0, size_t nrows,
                                const float* x, size_t x_stride, float* y, size_t y_stride,
                                size_t batch);
/* Several matrices times the SAME vectors in one pass (the Q, K and V, or the gate and up projections of a
 * decoder layer; no reference counterpart): ys[i][v*y_stride + r] = sum_c ws[i][r, c] * x[v*x_stride + c].  The
 * matrices share type and column count.  With a column count that is a multiple of 256 the vectors' fixed-point
 * planes are made once and one persistent launch of the tensor-core batch kernel walks up to 8 matrices (also for
 * one vector); otherwise it is one vx_gemv_q_rows per matrix.  Same arithmetic and results as the single calls. */
VX_API vx_status vx_gemv_q_multi(vx_context* ctx, const vx_qweights* const* ws, size_t n_matrices, const float* x,
                                 size_t x_stride, float* const* ys, size_t y_stride, size_t batch);

/* ------------------------------------------------- several GPUs, one process each ---- */
/* No reference counterpart (vortx knows one device ordinal, src/linalg/gemm.rs:353).
 * A row-sharded GEMV needs every rank's slab of y on every GPU.  Instead of a collective after
 * the kernel, vx_gemv_q_rows_scatter stores each finished row into the peers' y buffers as
 * well (plain stores over NVLink; nothing is loaded from a peer), and vx_peer_barrier tells
 * every rank when all slabs have landed.  Peer buffers are mapped with CUDA IPC:
 * export a vx_alloc'd buffer on its owner, pass the 64 bytes to the other processes by any
 * means, import them there. */
VX_API vx_status vx_ipc_export(vx_context* ctx, const void* device_ptr, void* handle64);
VX_API vx_status vx_ipc_import(vx_context* ctx, const void* handle64, void** device_ptr);
VX_API vx_status vx_ipc_release(vx_context* ctx, void* device_ptr);
/* y[r] and peer_y[i][r] (r < nrows, i < n_peers <= 7) all receive row row0 + r of W times x.  The
 * pointers are already advanced to where the slab belongs in each full-length y. */
VX_API vx_status vx_gemv_q_rows_scatter(vx_context* ctx, const vx_qweights* w, size_t row0, size_t nrows,
                                        const float* x, float* y, float* const* peer_y, size_t n_peers);
/* The same GEMV with the exchange fused into the kernel, for chains of dependent GEMVs (y of one is
 * x of the next): nothing runs between the links, no flag, fence or collective.
 * An exchange vector of n elements is vx_xvec_bytes(n) bytes of zero-initialised device memory,
 * 16-byte aligned, one per rank and mapped into the peers: a 256-byte header that only its owner
 * uses (word 0 = generation, how many times the vector has been written completely) and one 8-byte
 * pair {f32 value, u32 generation} per element.  Value and arrival mark travel in one 64-bit store.
 *   writer  row row0 + r of W times x (r < nrows) goes, tagged generation + 1, into element
 *           y_row0 + r * y_stride of y_xvec (this rank's) and of every peer_y_xvec[i] — stride 1
 *           for a contiguous slab of rows, the world size for rows dealt out in turn; into the
 *           plain y[r] as well unless y is null.  The grid's last block bumps the header.
 *   reader  with x_xvec non-null, x is that flagged vector (w's column count; the plain x is
 *           ignored): the weight stream starts at once, and each thread re-reads, for at most about
 *           0.2 s, the pairs that do not carry x_xvec's generation yet.
 * Every rank issues the same sequence of launches on the same vectors; a rank with no rows cannot
 * take part.  A vector is written again only after every rank has read it: a chain alternates
 * between two vectors (a rank can start link l + 1 only with all rows of link l, which every rank
 * produces after it has read its x).  vx_xvec_unpack turns a vector into plain f32, waiting the
 * same way; it is how a chain ends. */
VX_API size_t vx_xvec_bytes(size_t n);
VX_API vx_status vx_gemv_q_rows_exchange(vx_context* ctx, const vx_qweights* w, size_t row0, size_t nrows,
                                         const void* x_xvec, const float* x, float* y, void* y_xvec,
                                         void* const* peer_y_xvec, size_t n_peers, size_t y_row0,
                                         size_t y_stride);
VX_API vx_status vx_xvec_unpack(vx_context* ctx, const void* xvec, size_t n, float* out);

/* ------------------------------------------------ a list of GEMVs in one launch ---- */
/* No reference counterpart.  A decode step is a fixed list of matrix-vector products; launched one
 * by one, each pays its own launch, prologue and tail (about 4 us on B200, a fifth of a
 * 28672 x 8192 Q4_0 product).  A vx_gemv_batch runs the list in ONE persistent launch with one
 * continuous weight stream.  All entries share the quantisation type and the column count; the
 * fields of an entry mean what the arguments of vx_gemv_q_rows_exchange mean (x_xvec / y_xvec /
 * peers optional; with y_xvec null the entry is a plain product into y).
 * Entries run in order on every thread block but blocks are not synchronised with each other, so
 * an entry may only depend on an earlier one through an exchange vector: the earlier entry writes
 * it (y_xvec), the later one reads it (x_xvec) and waits pair by pair — on one GPU or across
 * GPUs alike.  A plain y of the list must not be the plain x of a later entry.  A vector may be
 * written again by a later entry only after every reader of its previous contents has read it;
 * a chain that alternates between two vectors satisfies this.
 * The list is uploaded once at creation (pointers are captured, not the data they point to) and
 * can be launched any number of times, also inside a CUDA graph. */
typedef struct vx_gemv_batch vx_gemv_batch;
typedef struct {
    const vx_qweights* w;
    size_t row0, nrows;         /* nrows >= 1                                       */
    const void* x_xvec;         /* flagged x, or NULL to read the plain x           */
    const float* x;
    float* y;                   /* plain rows, or NULL                              */
    void* y_xvec;               /* this rank's exchange vector, or NULL             */
    void* const* peer_y_xvec;   /* the same vector of every peer (n_peers entries)  */
    size_t n_peers;
    size_t y_row0, y_stride;    /* row r goes to element y_row0 + r * y_stride      */
    float* const* peer_y;       /* plain rows also stored here (n_peer_y buffers, as for
                                   vx_gemv_q_rows_scatter), or NULL                 */
    size_t n_peer_y;
    size_t x_seg_len, x_seg_stride, x_seg_first; /* with x_xvec: x is x_seg_len consecutive elements,
                                   from element x_seg_first, out of every x_seg_stride of the vector (a
                                   piece of every rank's slab); all 0: the vector's first cols elements.
                                   x_seg_len divides cols and is a multiple of 32; first and stride even */
} vx_gemv_op;
VX_API vx_status vx_gemv_batch_create(vx_context* ctx, const vx_gemv_op* ops, size_t n_ops,
                                      vx_gemv_batch** out);
VX_API vx_status vx_gemv_batch_launch(vx_context* ctx, const vx_gemv_batch* batch);
VX_API vx_status vx_gemv_batch_free(vx_context* ctx, vx_gemv_batch* batch);
/* Lists with HOST buffers, copies overlapped with the kernels.  The reference's callers keep their data in
 * host memory around a dispatch (tensors built from host matrices, `slow_read_buffer` after `synchronize`,
 * src/linalg/gemm.rs:378-426); a step is cut into stages so that the copies hide behind the kernels:
 *   stage i   copy up_bytes from up_host to up_device (skipped when 0), run the list, then, if barrier_flags
 *             is not NULL, a vx_peer_barrier over (barrier_flags, world, rank), then copy down_rows rows of
 *             down_width_bytes from down_device (rows down_device_pitch apart) to down_host (rows
 *             down_host_pitch apart; skipped when either count is 0).
 * Stage i + 1's copy up and stage i - 1's copy down run beside stage i's kernels, on two streams of the
 * context's own.  Host buffers should be page-locked (vx_host_alloc), or the copies do not overlap.
 * Returns when every stage's results are in host memory; work given to the context's stream before the call
 * is waited for first.  The lists must not be launched by anyone else meanwhile. */
typedef struct vx_host_stage {
    const vx_gemv_batch* batch;
    void* up_device;
    const void* up_host;
    size_t up_bytes;
    void* down_host;
    size_t down_host_pitch;
    const void* down_device;
    size_t down_device_pitch;
    size_t down_width_bytes;
    size_t down_rows;
    uint32_t* const* barrier_flags;
    size_t world, rank;
} vx_host_stage;
VX_API vx_status vx_gemv_batch_run_host(vx_context* ctx, const vx_host_stage* stages, size_t n_stages);
/* The same step recorded once (a CUDA graph over the three streams) and replayed: one runtime call per step
 * instead of a dozen, which matters once a step's kernels are shorter than those calls (0.1 ms on 8 GPUs).
 * Pointers and sizes are captured at creation; the host buffers MUST be page-locked.  create runs the step once.
 * run returns when every stage's results are in host memory. */
typedef struct vx_host_pipeline vx_host_pipeline;
VX_API vx_status vx_host_pipeline_create(vx_context* ctx, const vx_host_stage* stages, size_t n_stages,
                                         vx_host_pipeline** out);
VX_API vx_status vx_host_pipeline_run(vx_host_pipeline* pipeline);
VX_API vx_status vx_host_pipeline_free(vx_host_pipeline* pipeline);
/* Column-sharded GEMM: this rank's panel of C = A * B (out, lhs, rhs and shapes as for vx_gemm_f32
 * with VX_GEMM_TF32; out already advanced to the panel's first column, its row stride the full
 * width of C) computed by the tensor-core kernel, whose epilogue sends every 32 x 32 block of the
 * panel with tiled TMA stores to this GPU's C and to the same position of each peer's C (whole
 * 128-byte rows over NVLink, asynchronous to the tensor cores; nothing is loaded from a peer).
 * vx_peer_barrier afterwards tells every rank that all panels have landed.  One matrix, unit column
 * strides, 16-byte aligned bases and row pitches; anything else is VX_ERR_UNSUPPORTED (no fallback
 * here, the caller picks the collective form). */
VX_API vx_status vx_gemm_tf32_scatter(vx_context* ctx, float* out, const float* lhs, const float* rhs,
                                      const vx_shapes3* shapes, float* const* peer_out, size_t n_peers);
/* flags[r] (r < world <= 8) is rank r's sync block of 64 u32, zero-initialised: its own for
 * r == rank, a mapped peer pointer otherwise.  Stream-ordered: after all earlier work of this
 * context it announces this rank's next barrier number to every rank, then waits, on the device
 * and for at most about 0.2 s, until every rank has announced the same number (all ranks must
 * issue the same sequence of barriers; the count lives on the device, so a replayed CUDA graph
 * keeps advancing).  A wait that gives up surfaces as VX_ERR_DEVICE_TIMEOUT from the next
 * vx_synchronize.  One barrier orders "every rank has written" before "any rank reads"; a buffer
 * that is rewritten later needs its own ordering against the readers (a second barrier or a
 * second buffer). */
VX_API vx_status vx_peer_barrier(vx_context* ctx, uint32_t* const* flags, size_t world, size_t rank);

/* ------------------------------------------------------- a group of GPUs of one node ---- */
/* No reference counterpart.  One vx_group per context and rank (a process or thread per GPU): an NCCL
 * communicator for the collective forms, plus what the fused forms need (buffers every rank can store into,
 * mapped through CUDA IPC, and the arrival flags of vx_peer_barrier).  NCCL is loaded at run time
 * (libnccl.so.2, or the path in the environment variable VX_NCCL_LIBRARY); without it these entry points
 * return VX_ERR_COLLECTIVE for more than one rank.  Every rank makes the same calls in the same order.
 *   rank 0: vx_group_unique_id -> its 128 bytes reach the other ranks by any means (a file, a socket)
 *   all:    vx_group_create(ctx, world, rank, id) ... vx_group_destroy, with no work in flight. */
typedef struct vx_group vx_group;
VX_API vx_status vx_group_unique_id(void* id128);
VX_API vx_status vx_group_create(vx_context* ctx, size_t world, size_t rank, const void* id128, vx_group** out);
VX_API vx_status vx_group_destroy(vx_group* g);
VX_API vx_status vx_group_info(const vx_group* g, size_t* world, size_t* rank);
/* Collectives, stream-ordered on the context's stream.  all_gather: recv holds world x bytes_per_rank; send
 * NULL = in place (this rank's part already sits at recv + rank * bytes_per_rank). */
VX_API vx_status vx_group_all_gather(vx_group* g, const void* send, void* recv, size_t bytes_per_rank);
VX_API vx_status vx_group_broadcast(vx_group* g, void* buffer, size_t bytes, size_t root);
/* vx_peer_barrier over the group's own flags: after it, on this rank's stream, every rank's earlier peer stores
 * have landed here. */
VX_API vx_status vx_group_barrier(vx_group* g);
/* A zeroed buffer of `bytes` on every rank, each mapped into all the others: ptrs[r] (world entries) is the
 * pointer through which THIS process reaches rank r's buffer (ptrs[rank] its own).  Peer pointers are for
 * stores from this library's kernels only.  Collective; blocks until done. */
VX_API vx_status vx_group_peer_alloc(vx_group* g, size_t bytes, void** ptrs);
VX_API vx_status vx_group_peer_free(vx_group* g, void* const* ptrs);
/* Row-sharded GEMV: `slab` holds this rank's rows [row0, row0 + slab rows) of W; every finished row is stored at
 * float index row0 + r of the y of EVERY rank (y_all from vx_group_peer_alloc, y_offset bytes into each), then
 * the group's barrier.  After it, stream-ordered, the whole y is on this GPU.  x is replicated. */
VX_API vx_status vx_group_gemv_q(vx_group* g, const vx_qweights* slab, size_t row0, const float* x,
                                 void* const* y_all, size_t y_offset);
/* Column-sharded GEMM: C[m, n] = A[m, k] B[k, n], this rank computing columns [col0, col0 + ncols) from its
 * panel of B (rows rhs_stride floats apart) on the tensor cores, its epilogue storing every tile into the C of
 * every rank (c_all from vx_group_peer_alloc, row-major m x n), then the group's barrier.  A is replicated. */
VX_API vx_status vx_group_gemm_tf32(vx_group* g, const float* lhs, const float* rhs_panel, size_t m, size_t n,
                                    size_t k, size_t col0, size_t ncols, size_t rhs_stride, void* const* c_all);

/* --------------------------------------------------------------- reductions ---- */
/* Reduce::launch(backend, shapes, pass, variant, input, output) — src/linalg/reduce.rs:79-207 —
 * over the kernels of vortx-shaders/src/linalg/reduce.rs:19-367.  Only the w axis of `shape` is
 * walked (element i is in[i * w_stride]); the result is written to out[0].  f32 min / max start
 * from +-1e18 as the reference kernels do (reduce.rs:292-295). */
typedef enum {
    VX_REDUCE_SUM = 0,   /* ReduceVariant::Sum    — reduce_add_{f32,u32,i32}   */
    VX_REDUCE_PROD = 1,  /* ReduceVariant::Prod   — reduce_mul_*                */
    VX_REDUCE_MIN = 2,   /* ReduceVariant::Min    — reduce_min_*                */
    VX_REDUCE_MAX = 3,   /* ReduceVariant::Max    — reduce_max_*                */
    VX_REDUCE_SQNORM = 4 /* ReduceVariant::SqNorm — reduce_sq_norm (f32 only)   */
} vx_reduce_op;
typedef enum { VX_F32 = 0, VX_U32 = 1, VX_I32 = 2 } vx_dtype;
typedef enum {
    VX_REDUCE_ORDERED = 0, /* one 128-thread block in the reference kernel's order: bit-identical  */
    VX_REDUCE_WIDE = 1     /* many blocks + a fold over per-block partials held in scratch memory
                              the context owns; f32 sum / product / norm differ by rounding order  */
} vx_reduce_mode;
VX_API vx_status vx_reduce(vx_context* ctx, vx_reduce_op op, vx_dtype dtype, vx_reduce_mode mode,
                           const void* in, const vx_shape* shape, uint64_t cap_in, void* out);

/* No counterpart in the reference.  The VX_REDUCE_WIDE reduction for callers that must not
 * allocate at the moment of the call — a host that gave the whole device to its own arena at
 * start-up and forbids driver allocations afterwards, or a latency-critical loop that cannot
 * afford the device-wide stall a cudaMalloc may cause.  It needs no vx_context (creating one
 * allocates): work goes to `cuda_stream` (a cudaStream_t) of `device`, and the per-block partials
 * live in a fixed 4 KB array inside the library's device image instead of allocated scratch.
 *   - At most 67 108 864 elements (1024 partials x 65 536 elements per block); more is refused
 *     with VX_ERR_UNSUPPORTED.
 *   - The first call on each device looks up the array's device address and loads the code of every
 *     kernel the entry point can launch (any operation, any type); make that first call before any
 *     stream capture on that device.  Later calls on that device load and allocate nothing.
 *   - All calls share the one array: two calls whose kernels can overlap on the GPU (different
 *     streams, no dependency) race.  Nothing needs clearing between calls.
 * Results equal those of vx_reduce(.., VX_REDUCE_WIDE, ..): identical for integers and for
 * min / max; f32 sums, products and norms agree to rounding order (the two split the vector
 * into different numbers of blocks). */
VX_API vx_status vx_reduce_static(int32_t device, void* cuda_stream, vx_reduce_op op, vx_dtype dtype,
                                  const void* in, const vx_shape* shape, void* out);

/* -------------------------------------------------------- element-wise kernels ---- */
/* The `.call(pass, num_threads, shape_a, shape_b, a, b)` level of OpAssign — src/linalg/op_assign.rs:53-80
 * over gpu_add / gpu_sub / gpu_mul / gpu_div / gpu_copy (vortx-shaders/src/linalg/op_assign.rs:29-166)
 * and gpu_copy_with_offsets (:171-187): for every linear id of shape_a, decomposed over shape_a's
 * sizes, a[offset_a + it_a(id)] op= b[offset_b + it_b(id)].  shape_b carries zero strides where b
 * is broadcast. */
typedef enum { VX_OP_ADD = 0, VX_OP_SUB = 1, VX_OP_MUL = 2, VX_OP_DIV = 3, VX_OP_COPY = 4 } vx_op;
VX_API vx_status vx_op_assign(vx_context* ctx, vx_op op, float* a, const vx_shape* shape_a, uint64_t cap_a,
                              const float* b, const vx_shape* shape_b, uint64_t cap_b, uint32_t offset_a,
                              uint32_t offset_b);
/* contiguous / contiguous_with_offset — vortx-shaders/src/linalg/contiguous.rs:18-85, called from
 * src/linalg/contiguous.rs:20-129: dest[i] = src[offset + it(n,c,h,w)] with i walked in row-major
 * order of shape_src's sizes.  Elements are 4 bytes of any type. */
VX_API vx_status vx_contiguous(vx_context* ctx, void* dest, uint64_t cap_dest, const void* src,
                               const vx_shape* shape_src, uint64_t cap_src, uint32_t offset);
/* repeat — vortx-shaders/src/linalg/repeat.rs:15-43, called from src/linalg/repeat.rs:24-88:
 * result[it_r(id)] = source[it_s(id mod source sizes)]. */
VX_API vx_status vx_repeat(vx_context* ctx, float* result, const vx_shape* shape_result, uint64_t cap_result,
                           const float* source, const vx_shape* shape_source, uint64_t cap_source);

/* -------------------------------------------------------- packed-weight files ---- */
/* No reference counterpart beyond the GGML dimension convention vortx's layouts carry (GGML_IDS and
 * permute_ggml, src/shapes.rs:15-18, :261-265).  Reads GGUF containers (versions 2 and 3, little-endian):
 * the file is mapped, its tensor records are listed, and a Q4_0 / Q8_0 matrix (GGML types 2 / 8, whose
 * blocks are byte for byte this library's host block stream) goes straight from the mapping into
 * vx_qweights_upload.  A GGML tensor lists its innermost dimension first: ne[0] = columns, ne[1] = rows. */
typedef struct vx_wfile vx_wfile;
VX_API vx_status vx_wfile_open(const char* path, vx_wfile** out);
VX_API vx_status vx_wfile_close(vx_wfile* f);
VX_API vx_status vx_wfile_count(const vx_wfile* f, size_t* count);
/* Record `index`: name (truncated to name_cap - 1 characters), GGML type number, dimensions (unused ones 1)
 * and size in bytes (0 for a type this library cannot size).  Any output pointer may be NULL. */
VX_API vx_status vx_wfile_tensor(const vx_wfile* f, size_t index, char* name, size_t name_cap, uint32_t* ggml_type,
                                 uint32_t* n_dims, uint64_t ne[4], uint64_t* bytes);
VX_API vx_status vx_wfile_find(const vx_wfile* f, const char* name, size_t* index);
/* The tensor's bytes inside the mapping (valid until vx_wfile_close): F32 / F16 / Q4_0 / Q8_0. */
VX_API vx_status vx_wfile_data(const vx_wfile* f, size_t index, const void** data, uint64_t* bytes);
/* Uploads a Q4_0 / Q8_0 matrix as device weights (rows = ne[1], columns = ne[0]). */
VX_API vx_status vx_wfile_load_qweights(vx_context* ctx, const vx_wfile* f, size_t index, vx_qweights** out);

/* ------------------------------------------------------------------ checksum ---- */
/* No reference counterpart.  One read-only pass over a device buffer (16-byte aligned, a whole number of
 * 16-byte groups): *device_out receives the XOR of all its 32-bit words, word j of each group rotated
 * left by 8 j bits.  Stream-ordered.  It verifies an upload without a read-back (compare with the same
 * fold of the host bytes), and, as a kernel that only reads, it is the read-only HBM bandwidth probe of
 * the benchmark. */
VX_API vx_status vx_checksum_u32(vx_context* ctx, const void* device_ptr, size_t bytes, uint32_t* device_out);
/* The same fold over the device form of quantised weights (both planes and their zero padding). */
VX_API vx_status vx_qweights_checksum(vx_context* ctx, const vx_qweights* w, uint32_t* device_out);

/* ----------------------------------------------------------------- tuning ---- */
/* Integer knobs for experiments ("gemv.variant", "gemv.rows_per_warp", "gemm.tf32.stages"...).
 * Unknown keys return VX_ERR_INVALID_ARGUMENT.  Defaults are the shipped configuration. */
VX_API vx_status vx_set_option(vx_context* ctx, const char* key, int64_t value);
VX_API vx_status vx_get_option(const vx_context* ctx, const char* key, int64_t* value);

#ifdef __cplusplus
}
#endif
#endif /* VORTX_B200_H */
