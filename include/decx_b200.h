/*
 * decx_b200 -- C ABI of the B200 (sm_100a) dense-GEMM path.
 *
 * This is the boundary a DECX build binds to replace its BLAS-CUDA GEMM kernels.
 * Plain pointers and sizes only; no C++ or framework types.  All matrices are
 * row-major with a row pitch ("ld") counted in ELEMENTS of the matrix type
 * (an element of a complex matrix is one {re, im} pair).
 *
 * Every function returns 0 on success, a negative DECXB200_E* code for an invalid
 * argument or a missing capability, or a positive cudaError_t value.  Nothing in this
 * library calls exit(), throws, or falls back to a host computation.
 */
#ifndef DECX_B200_H_
#define DECX_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define DECXB200_API __attribute__((visibility("default")))
#else
#define DECXB200_API
#endif

/* element types; the values are de::_DATA_TYPES_FLAGS_
 * (reference: srcs/includes/DECX/classes/type_info.h:20-43) */
#define DECXB200_FP32 1
#define DECXB200_FP64 2
#define DECXB200_FP16 3
#define DECXB200_CPLXF 5
#define DECXB200_CPLXD 6

#define DECXB200_EINVAL (-1)       /* null pointer, zero extent, unknown dtype            */
#define DECXB200_EALIGN (-2)       /* fp16 operand pitch/base not 16-byte aligned (TMA)    */
#define DECXB200_EWORKSPACE (-3)   /* workspace missing, misaligned or too small           */
#define DECXB200_EDRIVER (-4)      /* cuTensorMapEncodeTiled unavailable / failed          */
#define DECXB200_ETOOLARGE (-5)    /* extent beyond what the entry point supports          */
#define DECXB200_EKERNEL (-6)      /* the kernel reported a time-out through its status word */

/*
 * Scratch bytes decxb200_gemm needs for one problem (0 for fp16 and fp64).
 * fp32:  tf32 (hi, lo) planes of A and B.
 * cplxf: (hi, lo) planes of A viewed as M x 2K reals and of the 2K x 2N real
 *        expansion of B.
 * cplxd: the 2K x 2N real expansion of B (doubles).
 * Replaces the planner-owned A-transpose scratch of the reference
 * (srcs/modules/BLAS/GEMM/CUDA/large_squares/common/cuda_GEMM_LS_planner.cu:125-127,156-163).
 */
DECXB200_API size_t decxb200_gemm_workspace_bytes(int dtype, uint32_t M, uint32_t N, uint32_t K);

/*
 * D = alpha * A * B + beta * C   on the current device, asynchronously on `stream`.
 *
 *   A: M x K (lda), B: K x N (ldb), C: M x N (ldc) or NULL, D: M x N (ldd); device pointers.
 *   alpha, beta: host pointers to one element of the accumulate type (float for fp32 and
 *                fp16, float[2] = {re, im} for cplxf); NULL means 1 (alpha) / 0 (beta).
 *                C is not read when it is NULL or beta == 0.
 *   workspace:   device scratch of at least decxb200_gemm_workspace_bytes(), 256-byte
 *                aligned; may be NULL for fp16.
 *   status:      device word the kernel writes a non-zero code to if one of its bounded
 *                waits expires (never expected); may be NULL.  Must be zero before the call.
 *
 * Replaces the uniform kernel-caller signature of the reference,
 * decx::blas::_cu_GEMM_kernel_ptr<T>
 * (srcs/modules/BLAS/GEMM/CUDA/large_squares/common/cuda_GEMM_LS_planner.cuh:64-69) and the
 * callers behind it (fp32/GEMM_fp32_callers.cuh:75-215, fp16/GEMM_fp16_callers.cuh:57-128,
 * 64b/GEMM_64b_callers.cuh:78-98).  fp16 accumulates in fp32 and stores fp16.
 * fp32 and cplxf run as 3xTF32 and keep fp32 accuracy.
 * fp64 and cplxd (the remaining cases of the reference's dtype switch, GEMM_LS.cu:335-345; kernels
 * large_squares/64b/GEMM_fp64_B64_kernels.cu:58, cplxd/GEMM_cplxd_B64_kernels.cu:60) run on the fp64 tensor
 * path (warp-level DMMA); their alpha / beta are host pointers to double (double[2] for cplxd) and `status`
 * is not used (the kernel has no waits that could expire).
 */
DECXB200_API int decxb200_gemm(int dtype, void* stream, uint32_t M, uint32_t N, uint32_t K,
                               const void* A, uint64_t lda, const void* B, uint64_t ldb,
                               const void* C, uint64_t ldc, void* D, uint64_t ldd,
                               const void* alpha, const void* beta,
                               void* workspace, size_t workspace_bytes, unsigned* status);

/*
 * Same, with the tuning knobs exposed (tests and the benchmark use them):
 *   cta_group: one of DECXB200_TILE_*: 0 = library default (a small cost model picks), 1 = one CTA per
 *              128x256 tile, 2 = CTA pair per 256x256 tile, 3 = CTA pair per 256x512 tile (fp16 only)
 *   max_ctas:  upper bound on the persistent grid (0 = number of SMs)
 */
#define DECXB200_TILE_AUTO 0
#define DECXB200_TILE_128x256 1
#define DECXB200_TILE_256x256 2
#define DECXB200_TILE_256x512 3
DECXB200_API int decxb200_gemm_ex(int dtype, void* stream, uint32_t M, uint32_t N, uint32_t K,
                                  const void* A, uint64_t lda, const void* B, uint64_t ldb,
                                  const void* C, uint64_t ldc, void* D, uint64_t ldd,
                                  const void* alpha, const void* beta,
                                  void* workspace, size_t workspace_bytes, unsigned* status,
                                  int cta_group, int max_ctas);

/*
 * Host-pointer form: A, B, C, D are HOST matrices (pinned memory gives full PCIe speed,
 * pageable memory works).  The call copies B once, then walks A and D in row blocks so that
 * the host->device copy of block i+1 and the device->host copy of block i-1 overlap the GEMM
 * of block i, on three library-owned streams of the current device.  It returns when D is
 * complete in host memory.
 *
 *   arena: DEVICE scratch of at least decxb200_gemm_host_arena_bytes(), 256-byte aligned.
 *          The library allocates no device memory itself: DECX's device memory pool (or any
 *          other allocator of the caller) provides it.
 *   has_c: whether a C operand with beta != 0 will be passed.
 *
 * This is the backend of the host-matrix overloads de::blas::cuda::GEMM(de::Matrix&, ...)
 * that the reference declares in srcs/includes/DECX/BLAS/BLAS.h:69-70 and never defines; it
 * covers what de::Memcpy (srcs/modules/core/data transmission/data_transmission.cu:105-180,
 * cudaMemcpy2DAsync honouring both pitches) plus the device GEMM plus de::Memcpy back would do.
 */
DECXB200_API size_t decxb200_gemm_host_arena_bytes(int dtype, uint32_t M, uint32_t N, uint32_t K, int has_c);
DECXB200_API int decxb200_gemm_host(int dtype, uint32_t M, uint32_t N, uint32_t K,
                                    const void* A, uint64_t lda, const void* B, uint64_t ldb,
                                    const void* C, uint64_t ldc, void* D, uint64_t ldd,
                                    const void* alpha, const void* beta,
                                    void* arena, size_t arena_bytes, unsigned* status);

/*
 * The host-pointer form sharded over several GPUs of this process (fp16, plain D = A.B; no counterpart in the
 * single-GPU reference -- it is what the host-matrix overloads de::blas::cuda::GEMM(de::Matrix&, ...), which the
 * reference declares in BLAS.h:69-70 and never defines, use when more than one GPU is visible).
 * Rows of A and D are dealt to the devices in whole 256-row tiles; every device moves ITS rows over ITS OWN
 * PCIe link (A up, D down, in row blocks pipelined with the GEMMs) and uploads only its share of B's rows;
 * the devices then complete each other's copy of B over NVLink from inside the first GEMM kernel
 * (decxb200_gemm_fp16_fetch: per-panel flags written by the upload streams gate the peer copies), so B crosses
 * PCIe once in total and never waits for a host-side collective.  Without peer access between the devices
 * each one uploads all of B itself.  Synchronous: returns when D is complete in host memory.
 *
 *   devices: CUDA ordinals, distinct; arenas[i]: device scratch ON devices[i], 256-byte aligned, at least
 *   decxb200_gemm_host_multi_arena_bytes() bytes each.  N must be a multiple of 8.  Pin the host matrices
 *   (portable pinning, so that every device sees them as pinned) for full PCIe speed.
 *   The caller's current device is restored before the call returns.
 */
DECXB200_API size_t decxb200_gemm_host_multi_arena_bytes(int dtype, int n_devices, uint32_t M, uint32_t N, uint32_t K);
/* The partition decxb200_gemm_host_multi uses, for inspection (arrays of n_devices entries, panel_end of 16; any
 * pointer may be NULL): rows of A / D per device and the height of its row blocks, the rows of B each device
 * uploads, and the column panels (exclusive ends) in which B is completed. */
DECXB200_API int decxb200_gemm_host_multi_plan(int n_devices, uint32_t M, uint32_t N, uint32_t K,
                                               uint32_t* row0, uint32_t* nrows, uint32_t* block_rows,
                                               uint32_t* piece0, uint32_t* piece_rows,
                                               uint32_t* n_panels, uint32_t* panel_end);
DECXB200_API int decxb200_gemm_host_multi(int dtype, int n_devices, const int* devices,
                                          uint32_t M, uint32_t N, uint32_t K,
                                          const void* A, uint64_t lda, const void* B, uint64_t ldb,
                                          void* D, uint64_t ldd, void* const* arenas, size_t arena_bytes);

/*
 * fp32 GEMM for callers that must not allocate.  (No counterpart in the reference, whose GEMM always
 * takes its scratch from the device memory pool.)
 *
 * Some code that wants an fp32 GEMM cannot obtain device scratch for it: a plug-in that runs inside a
 * host application whose own allocator has already claimed the GPU's memory, a latency-critical loop
 * that may not risk the implicit device synchronisation and the driver locks of cudaMalloc/cudaFree, or
 * a module that is only ever handed finished input and output buffers.  For them this entry point keeps
 * the scratch of the 3xTF32 path (the tf32 hi/lo planes of A and B) in a fixed array inside the library:
 * DECXB200_NOALLOC_SCRATCH_BYTES of device memory, held by every GPU context that loads the library for
 * as long as the process lives.  The caller passes only inputs and outputs; the call itself uses no
 * cudaMalloc, cudaFree or any other allocating routine.
 *
 *   Same meaning as decxb200_gemm(DECXB200_FP32, ...): D = alpha * A * B + beta * C, device pointers,
 *   asynchronous on `stream`, `status` optional.
 *   Limit: decxb200_gemm_workspace_bytes(DECXB200_FP32, M, N, K) must not exceed
 *   DECXB200_NOALLOC_SCRATCH_BYTES (for example 1024 x 1024 x 1024 fits exactly); larger problems return
 *   DECXB200_ETOOLARGE and launch nothing.
 *   First use: the first call on each device looks up the array's device address (with that device
 *   current) and remembers it.  Make that first call during set-up, before any stream capture begins.
 *   Sharing: every call on a device uses the same array, and the array keeps what the previous call
 *   left in it; each call clears the part it is going to use before writing its planes.  Two calls that
 *   overlap on the GPU (different streams, or different host threads without ordering) race on it:
 *   order them on one stream or with events.
 */
#define DECXB200_NOALLOC_SCRATCH_BYTES (16u << 20)
DECXB200_API int decxb200_gemm_fp32_noalloc(void* stream, uint32_t M, uint32_t N, uint32_t K,
                                            const void* A, uint64_t lda, const void* B, uint64_t ldb,
                                            const void* C, uint64_t ldc, void* D, uint64_t ldd,
                                            const void* alpha, const void* beta, unsigned* status);

/*
 * Matrix-vector products: the Vector overloads of de::blas::cuda::GEMM
 * (reference: srcs/includes/DECX/BLAS/BLAS.h:79-80, drivers srcs/modules/BLAS/GEMM/CUDA/VMM.cu:55-184, kernels
 * extreme_shapes/VMM_fp32.cu, VMM_fp16.cu).  A is rows x cols, row-major, lda elements per row; device pointers.
 *   trans == 0:  y[rows] = A . x[cols]      (Matrix x Vector)
 *   trans == 1:  y[cols] = x[rows] . A      (Vector x Matrix)
 * dtype DECXB200_FP32 (fp32 result) or DECXB200_FP16 with the reference's three accumulation levels
 * (srcs/common/Classes/classes_util.h:287-300): L1 = fp32 arithmetic and an fp32 RESULT vector, L2 = fp32
 * arithmetic and an fp16 result, L3 = fp16 arithmetic throughout and an fp16 result.
 * One pass over A; skinny shapes cut the reduction into slices whose partial vectors go through `workspace`
 * (decxb200_gemv_workspace_bytes, 16-byte aligned; without it the call still works, one slice, slower) and are
 * added in slice order: results do not depend on timing.  Asynchronous on `stream`.
 */
#define DECXB200_FP16_ACCU_L1 0
#define DECXB200_FP16_ACCU_L2 1
#define DECXB200_FP16_ACCU_L3 2
DECXB200_API size_t decxb200_gemv_workspace_bytes(int dtype, int fp16_accu, int trans, uint32_t rows, uint32_t cols);
DECXB200_API int decxb200_gemv(int dtype, int fp16_accu, int trans, void* stream, uint32_t rows, uint32_t cols,
                               const void* A, uint64_t lda, const void* x, void* y,
                               void* workspace, size_t workspace_bytes);

/*
 * dst (cols x rows, ldd) = transpose of src (rows x cols, lds); elements of 1, 2, 4, 8 or 16 bytes; pitches in
 * elements.  Reference: de::cuda::Transpose, srcs/modules/BLAS/Basic_process/transpose/transpose.cu:50-101.
 */
DECXB200_API int decxb200_transpose(int elem_bytes, void* stream, uint32_t rows, uint32_t cols,
                                    const void* src, uint64_t lds, void* dst, uint64_t ldd);

/*
 * Element type cast of a pitched rows x cols matrix.  Reference: de::cuda::TypeCast,
 * srcs/modules/BLAS/Basic_process/type_cast/GPU_Matrix_type_cast.cu:38-85 (fp32<->fp64, int32->fp32); the
 * fp32<->fp16 pair has no counterpart there -- the reference can only make fp16 operands element by element on
 * the host (de::Float2Half).  Float narrowing rounds to nearest even; fp32->int32 rounds to nearest even and
 * saturates.
 */
#define DECXB200_CAST_F32_F16 0
#define DECXB200_CAST_F16_F32 1
#define DECXB200_CAST_F32_F64 2
#define DECXB200_CAST_F64_F32 3
#define DECXB200_CAST_I32_F32 4
#define DECXB200_CAST_F32_I32 5
DECXB200_API int decxb200_cast2d(int kind, void* stream, uint32_t rows, uint32_t cols,
                                 const void* src, uint64_t lds, void* dst, uint64_t ldd);

/*
 * fp32 2-D convolution as im2col + one 3xTF32 GEMM: the consumer of the GEMM core in DECX's NN module
 * (reference: de::nn::cuda::Conv2D, srcs/modules/NN/convolution/CUDA/fp32/Conv2D.cu:57-131, planner
 * cuda_conv2D_fp32_im2col_planner.cu:200-300, kernels im2col_fp32.cu and im2col_GEMM_fp32.cu).  Tensors are stored
 * channels-innermost, element (y, x, c) at base[(y * wpitch + x) * dpitch + c] (srcs/common/Classes/Tensor.h:59-82).
 * Like the reference it is a cross-correlation (no kernel flip):
 *     dst(y, x, t) = sum_{i, j, c} src(y*sy + i - py, x*sx + j - px, c) * kernel_t(i, j, c)
 *   extend = DECXB200_EXTEND_NONE:      py = px = 0,  OH = (H - kh + 1) / sy,  OW = (W - kw + 1) / sx
 *   extend = DECXB200_EXTEND_CONSTANT:  py = kh / 2, px = kw / 2, zeros outside src,  OH = H / sy,  OW = W / sx;
 *                                       source rows at and below OH * sy also read as zeros, as in the reference
 *                                       (im2col_fp32.cu:132)
 * (the values of de::extend_label, srcs/includes/DECX/basic_proc/VectorProc.h:22-26).  kernels: n_kernels tensors of
 * kh x kw x C, tensor t at kernels + t * kernel_stride floats.  dst: OH x OW x n_kernels with dst_wpitch (0 = OW) and
 * dst_dpitch >= n_kernels; positions x in [OW, dst_wpitch) of the dst rows are left alone or written with zeros.
 * All device pointers; asynchronous on `stream`.  Two forms: when n_kernels and dst_dpitch are multiples of 4 and dst
 * is 16-byte aligned (DECX's tensors are) the GEMM kernel reads its operand tiles straight out of tf32 planes of the
 * zero-bordered source with 4-D TMA boxes (implicit GEMM; workspace = those planes + the packed kernels, about twice
 * the source); otherwise the tf32 planes of the im2col matrix are written to the workspace first.  The workspace
 * query takes the destination pitch for that reason; a misaligned dst with a multiple-of-4 pitch needs the size the
 * query returns for an odd pitch.  de::nn::cuda::Conv2D of the C++ drop-in (include/DECX/nn/convolution.h) is built
 * on this entry point; it is also what the reference's conv2D_im2col_fp32_caller would bind.
 */
#define DECXB200_EXTEND_NONE 0
#define DECXB200_EXTEND_CONSTANT 2
DECXB200_API int decxb200_conv2d_fp32_out_dims(uint32_t H, uint32_t W, uint32_t kh, uint32_t kw, uint32_t sx, uint32_t sy,
                                               int extend, uint32_t* OH, uint32_t* OW);
DECXB200_API size_t decxb200_conv2d_fp32_workspace_bytes(uint32_t H, uint32_t W, uint32_t C, uint32_t kh, uint32_t kw,
                                                         uint32_t n_kernels, uint32_t sx, uint32_t sy, int extend,
                                                         uint32_t dst_wpitch, uint32_t dst_dpitch /* 0 = n_kernels */);
DECXB200_API int decxb200_conv2d_fp32(void* stream, const void* src, uint32_t H, uint32_t W, uint32_t C,
                                      uint32_t src_wpitch, uint32_t src_dpitch,
                                      const void* kernels, uint32_t kh, uint32_t kw, uint32_t n_kernels,
                                      uint32_t kernel_wpitch, uint32_t kernel_dpitch, uint64_t kernel_stride,
                                      void* dst, uint32_t dst_wpitch, uint32_t dst_dpitch,
                                      uint32_t sx, uint32_t sy, int extend,
                                      void* workspace, size_t workspace_bytes, unsigned* status);

/*
 * Peer-visible device buffers for the row-sharded multi-GPU GEMM (one process per GPU).
 * The owner of the result allocates D with decxb200_ipc_alloc and exports a 64-byte handle;
 * every other rank opens it and passes `peer_ptr + its row offset` as the D argument of
 * decxb200_gemm, so the GEMM epilogue stores its rows straight into the owner's memory over
 * NVLink ("C gathered on the owner" with no separate gather step).  The reference is
 * single-GPU (no cudaSetDevice / peer / collective call anywhere in its sources), so these
 * have no counterpart there.
 */
DECXB200_API int decxb200_ipc_alloc(size_t bytes, void** dptr);

/*
 * fp16 GEMM whose B operand is still arriving (row-sharded multi-GPU GEMM; no counterpart in the
 * single-GPU reference).  B is a full K x N row-major replica in this GPU's memory that another
 * stream fills column panel by column panel (panel i = columns [panel_col_end[i-1], panel_col_end[i]),
 * at most 16 panels, the last end = N, the others multiples of 256; of 512 when the 256x512 tile is forced).  After panel i's data, that stream
 * writes `epoch` to panel_flags[i] (decxb200_write_flag_async).  ONE kernel launch computes D = A.B: it
 * walks the tiles panel by panel and its loader waits -- bounded, then status word 0x106 -- for a panel's
 * flag before it touches that panel, so the transfer of B overlaps the tiles of the panels before it.
 * Epochs must increase from one use of the flags to the next.
 */
DECXB200_API int decxb200_gemm_fp16_panels(void* stream, uint32_t M, uint32_t N, uint32_t K,
                                           const void* A, uint64_t lda, const void* B, uint64_t ldb,
                                           void* D, uint64_t ldd, unsigned* status,
                                           uint32_t n_panels, const uint32_t* panel_col_end,
                                           const unsigned* panel_flags, unsigned epoch, int max_ctas,
                                           int tile /* DECXB200_TILE_AUTO or DECXB200_TILE_256x512 */);
/*
 * The same product with the transfer of B fused into the kernel (row-sharded multi-GPU GEMM, one call per GPU;
 * no counterpart in the single-GPU reference).  `B` is this GPU's replica of the K x N operand; at the call it
 * may hold nothing yet.  Besides its loader, MMA and epilogue warps every CTA runs "courier" warps that walk
 * `jobs` in order: each job is a piece of B (rows x columns of one panel) that lies, or will lie, in memory
 * this GPU can address -- the owner's B or another GPU's replica, both laid out like the local one (row pitch
 * ldb) -- and is copied into the replica with 16-byte peer loads.  Pieces are counted per panel; when a panel is
 * complete its word in ready_flags is set to `epoch` and the tiles of that panel start.  A job with
 * publish = 1 is a piece this GPU is the first to hold outside the owner: once all publishing pieces of a
 * panel have landed, pub_flags[panel] is set to `epoch`, and the other GPUs' jobs name that word as their
 * `gate`.  So the owner sends every byte of B once (scatter) and the GPUs complete each other (all-gather),
 * inside the same launch that multiplies and that stores D into the owner's memory.
 *
 *   A job may also PUSH: dst names another GPU's replica and src is local; when all of the job is stored, `notify`
 *   (that GPU's publish flag for the panel) is set.  Posted stores need no request towards the sender, so the
 *   owner -- whose inbound link is busy receiving D -- scatters B by pushing, and the receivers list the pushed
 *   piece as a rows == 0 job gated on their own publish flag.  A GPU whose jobs all push (the owner) passes NULL
 *   for ready_flags / pub_flags and runs ungated.
 *   With publish = DECXB200_FETCH_MULTICAST a push job's dst and notify are addresses inside an NVLink MULTICAST
 *   mapping of all the GPUs' replicas and flag words (what CUDA's multicast objects / torch symmetric memory's
 *   multicast_ptr provide): the couriers store with multimem.st, the switch writes every store into all bound
 *   GPUs, and the flag of every GPU is raised with one multimem.red (max).  The owner then sends B over its link
 *   once, nobody fetches pieces from anybody, and the receivers' job lists hold only rows == 0 jobs gated on
 *   their own flags.
 *   jobs:      HOST array, copied by the call.  gate == NULL: the source is readable now.  rows == 0: a piece
 *              that something else writes into the replica (a copy engine); the courier only waits for its
 *              gate and counts it.  Every panel needs at least one job.  col0, cols: multiples of 8.
 *   scratch:   device memory, 256-byte aligned, decxb200_fetch_scratch_bytes(n_jobs) bytes (counters, a timing
 *              record, the job table).  After the kernel, bytes [256, 512) hold 32 uint64 in ns of the GPU's
 *              global timer: [i] when panel i was complete, [16] kernel start, [17] kernel end, [18] total time
 *              the tile loaders waited for panels, [19] how many such waits.
 *   ready_flags, pub_flags: device words, one per panel; other GPUs must be able to read pub_flags.
 *   n_jobs == 0: this GPU already holds B (the owner); ready_flags may then be NULL (no gating at all).
 *   All waits are bounded: status 0x106 (a panel never completed) or 0x107 (a gate never opened).
 *   Epochs must increase from one use of the flags to the next.
 */
#define DECXB200_FETCH_MULTICAST 2
typedef struct decxb200_fetch_job {
    const void* src;
    const unsigned* gate;
    void* dst;                 /* NULL: pull into the local replica; else PUSH: the target GPU's replica */
    unsigned* notify;          /* push jobs: word in the target's memory set to `epoch` when the job is complete */
    uint32_t row0, rows;
    uint32_t col0, cols;
    uint32_t panel;
    uint32_t publish;          /* pull jobs: 0 / 1; push jobs: 0 or DECXB200_FETCH_MULTICAST */
} decxb200_fetch_job;
DECXB200_API size_t decxb200_fetch_scratch_bytes(uint32_t n_jobs);
DECXB200_API int decxb200_gemm_fp16_fetch(void* stream, uint32_t M, uint32_t N, uint32_t K,
                                          const void* A, uint64_t lda, void* B, uint64_t ldb,
                                          void* D, uint64_t ldd, unsigned* status,
                                          uint32_t n_panels, const uint32_t* panel_col_end,
                                          unsigned* ready_flags, unsigned* pub_flags, unsigned epoch,
                                          const decxb200_fetch_job* jobs, uint32_t n_jobs,
                                          void* scratch, size_t scratch_bytes, int max_ctas, int tile);
/*
 * The same call with a staging area for D (device memory of THIS GPU, 16-byte aligned, decxb200_fetch_d_stage_bytes()
 * bytes; NULL = decxb200_gemm_fp16_fetch).  For a D that lives in another GPU's memory: the epilogue of a 256 x 512
 * tile stores its boxes into a ring of two tiles per CTA in the staging area (local, L2-resident) and releases the
 * accumulators at once; the courier warps copy each finished part to D with 16-byte stores while the next tile is
 * being multiplied.  Without it all CTAs of all GPUs finish their tiles together and their TMA stores reach the
 * owner's NVLink port as one burst that holds the accumulators (and so the next tile's MMAs) until it has drained.
 * Used with the 256 x 512 tile only; other tiles store D directly.
 */
DECXB200_API size_t decxb200_fetch_d_stage_bytes(void);
DECXB200_API int decxb200_gemm_fp16_fetch_staged(void* stream, uint32_t M, uint32_t N, uint32_t K,
                                          const void* A, uint64_t lda, void* B, uint64_t ldb,
                                          void* D, uint64_t ldd, unsigned* status,
                                          uint32_t n_panels, const uint32_t* panel_col_end,
                                          unsigned* ready_flags, unsigned* pub_flags, unsigned epoch,
                                          const decxb200_fetch_job* jobs, uint32_t n_jobs,
                                          void* scratch, size_t scratch_bytes, int max_ctas, int tile,
                                                 void* d_stage, size_t d_stage_bytes);
/* 2-D copy by the copy engines between any two device buffers this process can address (peer mappings
 * included): `rows` rows of `width_bytes`, rows dpitch / spitch bytes apart.  cudaMemcpy2DAsync. */
DECXB200_API int decxb200_copy2d_async(void* stream, void* dst, size_t dpitch, const void* src, size_t spitch,
                                       size_t width_bytes, size_t rows);
/* Stream-ordered 32-bit store (cuStreamWriteValue32): no kernel, so it cannot be starved of an SM. */
DECXB200_API int decxb200_write_flag_async(void* stream, unsigned* flag, unsigned value);
DECXB200_API int decxb200_ipc_free(void* dptr);
DECXB200_API int decxb200_ipc_export(void* dptr, unsigned char handle[64]);
DECXB200_API int decxb200_ipc_open(const unsigned char handle[64], void** peer_ptr);
DECXB200_API int decxb200_ipc_close(void* peer_ptr);

/* Number of kernels the last decxb200_gemm* call of this thread launched (pre-passes included). */
DECXB200_API int decxb200_last_launch_count(void);

/* Which GEMM kernel the last call of this thread launched: 100*KIND + 10*CTAS + NACC
 * (KIND 0 = fp16, 1 = 3xTF32; CTAS = CTAs per tile; NACC = 256-column accumulators per tile), + 1000 when the kernel
 * carried courier warps, + 5000 / + 6000 for the 128 x 64 / 128 x 128 tiles of small 3xTF32 problems and of
 * convolutions with few kernels, + 20000 when the kernel ran as an implicit-GEMM convolution;
 * e.g. 22 = fp16 256x512 pair tile, 121 = 3xTF32 256x256 pair tile, 5111 = 3xTF32 128x64 tile. */
DECXB200_API int decxb200_last_kernel_variant(void);

/* Tensor maps (TMA descriptors) are cached per host thread by (address, extents, pitch, box); these are the
 * calling thread's counts of look-ups served from the cache and of fresh cuTensorMapEncodeTiled calls. */
DECXB200_API void decxb200_tensor_map_cache_stats(unsigned long long* hits, unsigned long long* misses);

/* Tuning aid.  With DECXB200_STATS=1 in the environment the GEMM kernels of the current device add to a 32-word
 * timing record (ns of the GPU's global timer): [18] / [19] time and count of loader waits for panel flags,
 * [20] time the MMA-issuing threads waited for operands, [21] for a free accumulator, [22] their whole tile
 * loops, [23] how many of them were counted.  This call copies the record out (after the kernels launched so far
 * have finished) and clears it. */
DECXB200_API int decxb200_debug_stats(unsigned long long out[32]);

/* Static description of an error code returned by this library. */
DECXB200_API const char* decxb200_strerror(int code);

/* Library version, "major.minor". */
DECXB200_API const char* decxb200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* DECX_B200_H_ */
