/*
 * lsg.h — C ABI of the B200 (sm_100a) quantized-GEMM library.
 *
 * Every entry point takes plain pointers and sizes, launches asynchronously on
 * the CUDA stream it is given (a cudaStream_t passed as void*), never
 * allocates or frees device memory unless its comment says so, and returns an
 * lsg_status (0 on success, negative on error).  The text of the last error of
 * the calling thread is available from lsg_last_error().  No C++ exception
 * crosses this boundary.
 *
 * Each declaration cites the interface of the reference project
 * (kkontosis/LayerStoRmGemmKernels, paths relative to its root) that it
 * replaces.
 */
#ifndef LSG_H_
#define LSG_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define LSG_API __attribute__((visibility("default")))
#else
#define LSG_API
#endif

/* ------------------------------------------------------------------------ */
/* Status codes                                                             */
/* ------------------------------------------------------------------------ */
typedef enum lsg_status {
    LSG_OK = 0,
    LSG_ERR_INVALID = -1,     /* bad argument (shape, divisibility, null pointer) */
    LSG_ERR_UNSUPPORTED = -2, /* type / dtype / mode not implemented             */
    LSG_ERR_WORKSPACE = -3,   /* workspace missing or too small                  */
    LSG_ERR_CUDA = -4,        /* a CUDA runtime call failed                      */
    LSG_ERR_ALIGNMENT = -5,   /* a pointer is not aligned as required            */
    LSG_ERR_DEVICE_WAIT = -6  /* a kernel gave up on a bounded device-side wait  */
} lsg_status;

/* Last error message of the calling thread ("" when none). */
LSG_API const char* lsg_last_error(void);

/* Library version string. */
LSG_API const char* lsg_version(void);

/* Reads and clears the device-side status word of the current device.  Kernels
 * that wait on an mbarrier do so with a time limit; when the limit runs out
 * they record a non-zero code here and return instead of spinning.  This call
 * synchronizes the device.  *code receives 0 when no kernel reported. */
LSG_API int lsg_device_status(int* code);

/* Limit of the device-side waits of the decode mat-vec kernels and of lsg_ep_barrier, in SM
 * clock cycles, process-wide (default 4e8, about 0.2 s; 0 restores the default).  Codes a
 * wait that ran out leaves in the status word: 1 data did not land, 2 a pipeline stage was
 * not released, 3 tensor-core completion, 4 tensor memory, 5 slab table of the grouped
 * mat-vec too small, 6 cross-GPU barrier, 7 expert-parallel receive buffer overflow.  No counterpart in the reference (its kernels do not wait). */
LSG_API int lsg_set_wait_limit_cycles(long long cycles);

/* Failure-path test hook: from now on the first CTA of every decode mat-vec launch leaves out
 * pipeline slab `slab` (it is neither loaded nor published), so that the consumers of that
 * slab run into the wait limit, record code 1 and return; slab < 0 switches the hook off.
 * The output of such a launch is incomplete by construction.  No counterpart in the
 * reference. */
LSG_API int lsg_test_mmvq_drop_slab(int slab);

/* ------------------------------------------------------------------------ */
/* GGUF weight types                                                        */
/* ids 0..6 replace: enum class GgufType,                                   */
/*   csrc/sm120/gemm/gguf/gguf_dequant_gemm.h:23-31                         */
/* id 7 (Q4_0) has no counterpart in the reference; it is appended so the   */
/* reference ids keep their meaning.                                        */
/* ------------------------------------------------------------------------ */
typedef enum lsg_gguf_type {
    LSG_GGUF_Q2_K = 0,
    LSG_GGUF_Q3_K = 1,
    LSG_GGUF_Q4_K = 2,
    LSG_GGUF_Q5_K = 3,
    LSG_GGUF_Q6_K = 4,
    LSG_GGUF_Q8_0 = 5,
    LSG_GGUF_MXFP4 = 6,
    LSG_GGUF_Q4_0 = 7
} lsg_gguf_type;

typedef enum lsg_dtype {
    LSG_DTYPE_BF16 = 0, /* what the reference always writes */
    LSG_DTYPE_F32 = 1,  /* extension: un-rounded accumulator, for parity checks */
    LSG_DTYPE_F16 = 2
} lsg_dtype;

/* Values per packed block (32 or 256); 0 for an unknown type.
 * Replaces gguf_block_values, csrc/sm120/gemm/gguf/gguf_dequant_gemm.cu:292-294 */
LSG_API int lsg_gguf_block_values(int type);

/* Bytes per packed block; 0 for an unknown type.
 * Replaces gguf_block_bytes, csrc/sm120/gemm/gguf/gguf_dequant_gemm.cu:296-307 */
LSG_API int lsg_gguf_block_bytes(int type);

/* ------------------------------------------------------------------------ */
/* Q8_1 activation quantizer                                                */
/* ------------------------------------------------------------------------ */

/* bf16 x[M,K] -> M*(K/32) blocks of 36 bytes {fp16 d, fp16 sum, int8 q[32]}.
 * K must be a multiple of 32.  Bit-exact with the reference kernel.
 * Replaces gguf_quantize_q8_1_cuda, csrc/sm120/gemm/gguf/gguf_mmvq.cu:124-128
 * (kernel quantize_bf16_to_q8_1, same file :42-63). */
LSG_API int lsg_quantize_q8_1(const void* x_bf16, void* q8_1_out, int M, int K, void* stream);

/* ------------------------------------------------------------------------ */
/* GGUF mmvq: C[M,N] = Q8_1(A[M,K]) . decode(B[N,K])^T  (decode GEMV)       */
/* ------------------------------------------------------------------------ */

/* Mirrors struct GgufMmvqParams, csrc/sm120/gemm/gguf/gguf_mmvq.h:21-27,
 * plus out_dtype. */
typedef struct lsg_gguf_mmvq_params {
    int M, N, K;
    const void* A; /* [M,K] bf16, row-major, device                      */
    const void* B; /* [N,(K/QK)*block_bytes] packed weight, 16-B aligned */
    void* C;       /* [M,N] out_dtype, row-major, device                 */
    int type;      /* lsg_gguf_type                                      */
    int out_dtype; /* lsg_dtype: BF16 (reference behaviour) or F32       */
} lsg_gguf_mmvq_params;

/* Bytes of caller-provided scratch for the quantized activation:
 * M*(K/32)*36.  Replaces gguf_mmvq_workspace_bytes,
 * csrc/sm120/gemm/gguf/gguf_mmvq.cu:120-122. */
LSG_API size_t lsg_gguf_mmvq_workspace_bytes(int M, int K);

/* Quantizes A to Q8_1 into `workspace`, then runs the integer mat-vec.
 * Any M >= 1 (rows are processed eight at a time).  K must be a multiple of
 * the type's block size.  Replaces launch_gguf_mmvq,
 * csrc/sm120/gemm/gguf/gguf_mmvq.cu:130-152. */
LSG_API int lsg_gguf_mmvq(const lsg_gguf_mmvq_params* p, void* workspace, size_t workspace_bytes,
                  void* stream);

/* Same mat-vec on activations that are already Q8_1 blocks (M*(K/32)*36 bytes
 * at xq).  p->A is ignored.  Exposed so that several projections sharing one
 * input quantize it once; no counterpart in the reference API (its kernel
 * gguf_mmvq_kernel, gguf_mmvq.cu:69-101, is file-local). */
LSG_API int lsg_gguf_mmvq_q8_1(const lsg_gguf_mmvq_params* p, const void* xq, void* stream);

/* Same operation as lsg_gguf_mmvq for callers that cannot allocate device memory -
 * a process on a fixed memory plan, a plug-in running inside someone else's runtime,
 * a decode loop that must never hit cudaMalloc.  The Q8_1 scratch is a device array
 * built into the library (held by every GPU that loads it, until exit), so only the
 * inputs and the output are passed.  M * (K/32) * 36 must not exceed
 * LSG_NOALLOC_MAX_Q8_1_BYTES, otherwise LSG_ERR_WORKSPACE.  The first call on a device
 * resolves the array's address: make it before any stream capture.  All calls share the
 * array (nothing in it needs clearing; each call rewrites what it reads), so calls whose
 * kernels may overlap on the GPU must be ordered by the caller.  The resolved address is
 * remembered per device ordinal and belongs to the device's primary context: call this only
 * under the primary context (what the runtime API and PyTorch use), and not across a
 * cudaDeviceReset.  This entry point has no counterpart in the reference, whose launchers
 * always take a caller workspace. */
#define LSG_NOALLOC_MAX_Q8_1_BYTES 147456
LSG_API int lsg_gguf_mmvq_noalloc(const lsg_gguf_mmvq_params* p, void* stream);

/* n projections in one call, with the results of executing them in order, each as
 * lsg_gguf_mmvq would.  Consecutive entries with the same M, K, type and out_dtype run as ONE
 * launch, up to six matrices per launch, their CTAs divided in proportion to the rows (one
 * prologue, one activation image per CTA and one pipeline fill instead of several): entries
 * with the same A (q, k and v of one hidden state; gate and up of one MLP input) always, and,
 * when the activations are quantized inside the mat-vec (M * K <= 32768), entries with
 * activations of their own as long as none of them reads or writes a buffer another entry of
 * the launch writes (byte ranges of A and C are compared).  A launch that shares no buffer
 * with the earlier entries of the call does not wait for the launch in front of it: its CTAs
 * start on the SMs that launch has left while its last CTAs still stream (only the first
 * launch of the call waits for the work in front of the call, and it releases the next launch
 * after that wait; the others wait before they exit, so the call still completes in stream
 * order).  An entry that reads an earlier entry's result, or writes a buffer an earlier entry
 * uses, waits as before.  LSG_MMVQ_BATCH_OVERLAP=0 in the environment switches both off.
 * Results are the bits of the separate calls.  Workspace:
 * lsg_gguf_mmvq_batch_workspace_bytes(p, n) (the largest Q8_1 image of the batch).  The
 * reference launches one kernel per projection (launch_gguf_mmvq,
 * csrc/sm120/gemm/gguf/gguf_mmvq.cu:130-152). */
LSG_API size_t lsg_gguf_mmvq_batch_workspace_bytes(const lsg_gguf_mmvq_params* p, int n);
/* How lsg_gguf_mmvq_batch would run the batch, without launching anything (host arithmetic on
 * the parameter blocks only; no device needed): returns the number of launches and, for the
 * first `cap` of them, the first entry, the number of entries and the kind of each: 0 waits for
 * the launch in front of it, 1 is the first launch of a batch whose later launches need not
 * wait (it waits for the work in front of the call and releases the next launch after that),
 * 2 does not wait for the launch in front of it; + 4 when a quantizer launch precedes the
 * mat-vec (activations above the in-kernel quantizer's limit).  Output arrays may be null. */
LSG_API int lsg_gguf_mmvq_batch_plan(const lsg_gguf_mmvq_params* p, int n, int* first, int* count, int* kind,
                                     int cap);
LSG_API int lsg_gguf_mmvq_batch(const lsg_gguf_mmvq_params* p, int n, void* workspace,
                        size_t workspace_bytes, void* stream);

/* Same operation with the activations and the result in HOST memory: p->A and p->C
 * are host pointers (p->B stays on the device).  The call copies A into `workspace`,
 * runs the mat-vec there and copies C back, all enqueued on `stream`; it does not wait
 * for the stream.  Page-locked, 16-byte aligned host buffers are read and written by the
 * kernels themselves through their device alias (no DMA copy, nothing blocks the calling
 * thread); pageable ones go through cudaMemcpyAsync and follow its rules.  The
 * caller must not touch A or C until the stream has passed this call.  Workspace:
 * lsg_gguf_mmvq_host_workspace_bytes(M, N, K).  The reference has no host-memory
 * variant; this is the entry a host-side integration binds when its tensors live in
 * host memory (one call instead of copy, launch, copy). */
LSG_API size_t lsg_gguf_mmvq_host_workspace_bytes(int M, int N, int K);
LSG_API int lsg_gguf_mmvq_host(const lsg_gguf_mmvq_params* p, void* workspace, size_t workspace_bytes,
                       void* stream);

/* n projections in one call, executed in order, each as lsg_gguf_mmvq_host would.
 * Entries naming the same A, M and K as an earlier entry reuse its Q8_1 image (the q, k
 * and v projections of one hidden state quantize it once), and consecutive ones share a
 * launch as in lsg_gguf_mmvq_batch.  All activations must be in place when the call is made:
 * up to eight distinct ones are quantized by a single launch up front.  When, in addition,
 * every result goes straight to its page-locked buffer (M <= 4) and no entry's buffers meet
 * another's, entries of one shape share a launch whatever their input and the launches do not
 * wait for each other, as in lsg_gguf_mmvq_batch: a layer of seven projections is three
 * launches.  (A batch in which a C overlaps the A of a later entry is still executed in
 * order, with a quantizer launch in front of each group of projections.)  n <= 64.
 * Workspace: lsg_gguf_mmvq_host_batch_workspace_bytes(p, n), 256-byte aligned. */
LSG_API size_t lsg_gguf_mmvq_host_batch_workspace_bytes(const lsg_gguf_mmvq_params* p, int n);
LSG_API int lsg_gguf_mmvq_host_batch(const lsg_gguf_mmvq_params* p, int n, void* workspace,
                             size_t workspace_bytes, void* stream);

/* Launch geometry of the mmvq kernels, process-wide: consumer warps per CTA
 * (1..15), CTAs of one launch per SM, KiB per pipeline stage, and how many CTAs
 * (of this and of neighbouring launches in the stream) split an SM's shared
 * memory.  An argument <= 0 keeps the current value.  skip_math must be <= 0 in
 * the shipped library; a bench build (-DLSG_DEBUG_KNOBS) accepts 1, which makes
 * kernels stream the weights without doing the arithmetic (outputs are then
 * zeros).  Results do not depend on the geometry.  No counterpart in the reference (its grid is fixed: one CTA per
 * output channel, gguf_mmvq.cu:104-112). */
LSG_API int lsg_mmvq_set_tuning(int consumer_warps, int ctas_per_sm, int stage_kib,
                                int smem_share, int skip_math);

/* ------------------------------------------------------------------------ */
/* GGUF mmq: prefill GEMM on the tensor cores                               */
/* ------------------------------------------------------------------------ */

/* C[M,N] = Q8_1(A) . decode(B)^T for large M through tcgen05 (fp16 operands made from
 * the Q8_1 round trip of A and the dequantized weight, fp32 accumulation).
 * Replaces launch_gguf_mmq_mma, csrc/sm120/gemm/gguf/mmq_mma/mmq_mma_dispatch.cu:52-91
 * (no Python binding of its own in the reference; reached through the grouped operator).
 * Workspace: lsg_gguf_mmq_workspace_bytes(M, N, K) bytes, 256-byte aligned. */
LSG_API size_t lsg_gguf_mmq_workspace_bytes(int M, int N, int K);
LSG_API int lsg_gguf_mmq(const lsg_gguf_mmvq_params* p, void* workspace, size_t workspace_bytes,
                         void* stream);

/* C[M,N] = A[M,K] (bf16, unquantized) . dequant(B)^T on the tensor cores: the packed weights
 * are decoded to fp16 inside the kernel; each activation row is moved into fp16 range by a
 * power of two of its own (exact for bf16 values) and the output row scaled back, so no
 * activation precision is lost.  For Q4_K this replaces the legacy launch_q4k_dequant_gemm
 * (csrc/sm120/gemm/q4k/q4k_dequant_gemm.cu:354-380) and launch_q4k_cutlass_gemm
 * (csrc/sm120/gemm/q4k/q4k_cutlass_gemm.cu:305-343; the reference rounds the weights to bf16
 * for its wmma tiles, fp16 keeps three more bits); for every type it is the fast sibling of
 * lsg_gguf_dequant_gemm.  Workspace: lsg_gguf_gemm_bf16_workspace_bytes(M, N, K) bytes,
 * 256-byte aligned (the reference's two launchers take none; its Python operators allocate
 * their output the same way this library's bindings allocate the workspace). */
LSG_API size_t lsg_gguf_gemm_bf16_workspace_bytes(int M, int N, int K);
LSG_API int lsg_gguf_gemm_bf16(const lsg_gguf_mmvq_params* p, void* workspace, size_t workspace_bytes,
                               void* stream);

/* lsg_gguf_mmq fused with the all-gather of a column-split weight: this rank holds N of the
 * ldc output columns (a slab of packed weight rows) and stores every output tile into each
 * of the n_out matrices C_ptrs[i] (a DEVICE array of device pointers: this GPU's [M, ldc]
 * output and its peers', peer-mapped) at column offset col_offset.  After a barrier over the
 * ranks every rank holds the whole [M, ldc] product; no collective moves the data, the
 * stores travel over NVLink while the tensor cores work on the next tiles.  p->C is ignored.
 * No counterpart in the reference (it has no multi-GPU code). */
LSG_API int lsg_gguf_mmq_gather(const lsg_gguf_mmvq_params* p, void* const* C_ptrs, int n_out, int ldc,
                                int col_offset, void* workspace, size_t workspace_bytes, void* stream);
/* The same with an NVLink multicast address of the output (the address under which a store
 * reaches the [M, ldc] matrix of EVERY rank, e.g. the multicast pointer of a symmetric-memory
 * allocation; NULL = lsg_gguf_mmq_gather).  Above 2048 rows the epilogue then issues one
 * multimem.st per 16 bytes instead of n_out peer stores, so a rank sends its slab once and the
 * switch replicates it.  C_ptrs is still required (smaller calls use it). */
LSG_API int lsg_gguf_mmq_gather_mc(const lsg_gguf_mmvq_params* p, void* const* C_ptrs, int n_out, int ldc,
                                   int col_offset, void* multicast_ptr, void* workspace, size_t workspace_bytes,
                                   void* stream);

/* How the tensor-core GEMMs (lsg_gguf_mmq and the grouped GEMM's tensor-core route) obtain
 * their fp16 weights, process-wide:
 *   0  a preparation kernel expands the packed matrix into workspace first;
 *   1  (default) types with a register-staged decoder (Q4_K) are decoded inside the GEMM
 *      kernel and never expanded; the others as in 0;
 *   2  every type is decoded inside the GEMM kernel.
 * A negative mode restores the default (or the LSG_TC_FUSED environment variable).  Results
 * agree between the modes to the fp16 rounding of the weights.  No counterpart in the
 * reference. */
LSG_API int lsg_mmq_set_weight_path(int mode);

/* ------------------------------------------------------------------------ */
/* GGUF dequant GEMM (lossless-activation golden strategy)                  */
/* ------------------------------------------------------------------------ */

/* C[M,N] = A[M,K] (bf16) . dequant(B)^T with fp32 accumulation.
 * Replaces launch_gguf_dequant_gemm,
 * csrc/sm120/gemm/gguf/gguf_dequant_gemm.cu:309-325
 * (params struct gguf_dequant_gemm.h:33-39). */
LSG_API int lsg_gguf_dequant_gemm(const lsg_gguf_mmvq_params* p, void* stream);

/* Expands packed blocks to fp32: out[n_blocks * block_values].  Test helper;
 * replaces the per-type dequant_*_block device functions of csrc/formats/. */
LSG_API int lsg_gguf_dequant_blocks(const void* packed, float* out, int type, long long n_blocks,
                            void* stream);

/* ------------------------------------------------------------------------ */
/* GGUF grouped GEMM: one MoE projection over E experts                     */
/* ------------------------------------------------------------------------ */
enum { LSG_GGUF_STRATEGY_DEQUANT = 0, LSG_GGUF_STRATEGY_INT = 1 };
/* replaces enum GgufGroupedStrategy, csrc/sm120/gemm/gguf/gguf_grouped_gemm.h:38-41 */
enum { LSG_GGUF_FORCE_AUTO = 0, LSG_GGUF_FORCE_MMVQ = 1, LSG_GGUF_FORCE_MMQ = 2,
       LSG_GGUF_FORCE_HOSTLOOP = 3 };
/* replaces GgufGroupedIntForce (gguf_grouped_int.h:100-104) and the binding's force
 * argument (csrc/bindings_python.cu:552,594-602) */

/* Mirrors struct GgufGroupedGemmKernelParams, gguf_grouped_gemm.h:43-55, plus out_dtype. */
typedef struct lsg_gguf_grouped_gemm_params {
    int type;                      /* lsg_gguf_type, shared by all experts           */
    int strategy;                  /* LSG_GGUF_STRATEGY_*                            */
    int num_experts;
    int N;                         /* output columns                                 */
    int K;                         /* input columns                                  */
    const void* A_base;            /* [total_tokens,K] bf16, rows grouped by expert  */
    void* D_base;                  /* [total_tokens,N] out_dtype                     */
    const int32_t* expert_offsets; /* [E+1] cumulative row counts, device            */
    const void* const* B_ptrs;     /* [E] packed weights, device array of device     */
                                   /* pointers; a null entry skips that expert       */
    int out_dtype;
} lsg_gguf_grouped_gemm_params;

/* Replaces gguf_grouped_gemm_workspace_bytes, gguf_grouped_gemm.cu:28-37.  The layout
 * differs from the reference's (it also holds this library's segment list), so callers
 * must size the workspace with this function. */
LSG_API size_t lsg_gguf_grouped_gemm_workspace_bytes(int total_tokens, int K, int num_experts);

/* Workspace that also holds the fp16 operands of the tensor-core path (N is needed for
 * that, which the reference's signature does not carry).  With only the smaller workspace
 * above, calls that would use tensor cores run the grouped mat-vec kernel instead. */
LSG_API size_t lsg_gguf_grouped_gemm_workspace_bytes_ex(int total_tokens, int K, int num_experts,
                                                        int N);

/* Replaces launch_gguf_grouped_gemm / _int_forced / _hostloop (gguf_grouped_gemm.cu:40-150).
 * Rows of experts that are empty or whose weight pointer is null are left untouched.
 * The Int strategy with force 0..2 never synchronizes with the host. */
LSG_API int lsg_gguf_grouped_gemm(const lsg_gguf_grouped_gemm_params* p, int total_tokens,
                                  void* workspace, size_t workspace_bytes, int force, void* stream);

/* Expert feed-forward block of a SwiGLU MoE layer in one call, over rows grouped by expert:
 *   D[T,H] = down( silu(gate(x)) * up(x) ),  silu(g) = g / (1 + exp(-g)),
 * with gate/up packed [I, H] and down packed [H, I] per expert.  Numerically the three
 * lsg_gguf_grouped_gemm calls (Int strategy, bf16 outputs) with the activation computed in
 * fp32 and stored as bf16 in between, which is how a caller of the reference's
 * gguf_grouped_gemm (csrc/bindings_python.cu:552-611) builds the block; the reference fuses
 * activation and quantizer only on its NVFP4 path (launch_silu_mul_to_nvfp4_grouped).
 * Never synchronizes with the host.  Rows of experts without rows are untouched; all three
 * pointers of an expert that has rows must be valid.
 * With `perm` set the permute (gather) of the MoE layer is folded into the call: A_base is
 * then the UNPERMUTED token matrix [num_tokens, H] and row i of the block is token
 * perm[i] / top_k (perm as lsg_moe_permutation writes it); the routed rows are never written
 * to memory as bf16, the first operand preparation reads the tokens directly. */
typedef struct lsg_gguf_moe_ffn_params {
    int type;                        /* lsg_gguf_type of all three matrices            */
    int num_experts;
    int H;                           /* model width: K of gate/up, N of down           */
    int I;                           /* expert width: N of gate/up, K of down          */
    const void* A_base;              /* [total_tokens, H] bf16, rows grouped by expert */
    void* D_base;                    /* [total_tokens, H] out_dtype                    */
    const int32_t* expert_offsets;   /* [E+1], device                                  */
    const void* const* gate_ptrs;    /* [E] device array of device pointers            */
    const void* const* up_ptrs;
    const void* const* down_ptrs;
    int out_dtype;
    const int32_t* perm;             /* optional [total_tokens] sorted-row -> (token, slot) pair  */
    int top_k;                       /* slots per token (with perm)                               */
} lsg_gguf_moe_ffn_params;
LSG_API size_t lsg_gguf_moe_ffn_workspace_bytes(int total_tokens, int H, int I, int num_experts);
LSG_API int lsg_gguf_moe_ffn(const lsg_gguf_moe_ffn_params* p, int total_tokens, void* workspace,
                             size_t workspace_bytes, void* stream);
/* Average rows per expert (total_tokens / num_experts, rounded down) up to which
 * lsg_gguf_moe_ffn composes the block from the grouped mat-vec kernels, whose results are
 * bit-identical to the reference's; above it the tensor-core kernels run (equal within the
 * tolerance of a GEMM with fp32 accumulation in another order).  Default 8, the batch at which
 * the reference leaves its mat-vec kernels (gguf_grouped_int.cu:918-919), or the environment
 * variable LSG_MOE_MATVEC_ROWS; -1 sends every batch to the tensor cores, which is faster from
 * about two rows per expert (128 experts of 2048 x 768, 64 / 128 tokens top-8: 0.33 -> 0.27 ms
 * and 0.47 -> 0.27 ms per layer).  Returns the previous value.  Process-wide, not synchronized
 * with calls in flight on other threads. */
LSG_API int lsg_gguf_moe_ffn_set_matvec_rows(int rows);

/* Ascending list of the experts that have rows, padded with -1 to `cap` entries.
 * Replaces build_active_expert_list, gguf_grouped_int.cu:156-187. */
LSG_API int lsg_build_active_expert_list(const int32_t* expert_offsets, int num_experts, int cap,
                                         int32_t* active_experts, void* stream);

/* m-tile t -> (expert, first row) for tiles of tile_m rows, padded with (-1, 0) to t_max.
 * Replaces build_mmq_tile_map, gguf_grouped_int.cu:46-66 (t_max as
 * gguf_grouped_mmq_tmax, gguf_grouped_int.h:91-95). */
LSG_API int lsg_build_mmq_tile_map(const int32_t* expert_offsets, int num_experts, int tile_m,
                                   int t_max, int32_t* tile_expert, int32_t* tile_mstart,
                                   void* stream);

/* ------------------------------------------------------------------------ */
/* Activation quantizers for the FP8 / NVFP4 paths                          */
/* ------------------------------------------------------------------------ */

/* FP8 (e4m3) block-scaled GEMM family.  D = sum over 128-wide K blocks of
 * scale_A[m,kb] * scale_B[n/128,kb] * (A8 . B8^T over the block).
 *   scale_A: fp32 [M, ceil(K/128)] M-major (what lsg_dynamic_fp8_quant writes with
 *            m_major_scales = 1); grouped: per expert, M-major inside the expert's rows,
 *            starting at expert_offsets[e] * ceil(K/128) floats
 *   scale_B: fp32 [ceil(K/128), ceil(N/128)] K-major (what lsg_weight_fp8_quant writes);
 *            grouped: one such matrix per expert, contiguous or through scale_B_ptrs
 * Replace launch_fp8_gemm / query_fp8_gemm_workspace_size (csrc/sm120/gemm/fp8/fp8_gemm.h:18-60,
 * fp8_gemm.cu), launch_fp8_grouped_gemm (fp8_grouped_gemm.cu:52-151; no host synchronisation
 * here) and launch_weight_fp8_quant (csrc/smxx/quant/weight_fp8_quant.cu:51-150, bit-exact).
 * K must be a multiple of 16.  M <= 4 with 16-byte aligned operands takes a mat-vec kernel
 * that needs no workspace (the role of fp8_blockscaled_gemv.cu:54-145 for M = 1). */
typedef struct lsg_fp8_gemm_params {
    int M, N, K;
    const void* A;         /* [M,K] e4m3 */
    const void* B;         /* [N,K] e4m3 */
    void* D;               /* [M,N] output_dtype */
    const void* scale_A;
    const void* scale_B;
    int output_dtype;      /* LSG_DTYPE_BF16, _F16 or _F32 */
} lsg_fp8_gemm_params;
LSG_API size_t lsg_fp8_gemm_workspace_bytes(int M, int N, int K);
LSG_API int lsg_fp8_gemm(const lsg_fp8_gemm_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* Mirrors struct Fp8GroupedGemmParams, csrc/sm120/gemm/grouped_gemm.h:84-105 (problem_sizes is
 * accepted and ignored: the row counts come from expert_offsets). */
typedef struct lsg_fp8_grouped_gemm_params {
    int num_experts, N, K;
    const void* A_base;
    const void* B_base;
    void* D_base;
    const void* scale_A_base;
    const void* scale_B_base;
    const int32_t* expert_offsets;
    const int32_t* problem_sizes;
    int output_dtype;
    const void* const* B_ptrs;
    const void* const* scale_B_ptrs;
} lsg_fp8_grouped_gemm_params;
LSG_API size_t lsg_fp8_grouped_gemm_workspace_bytes(int total_tokens, int num_experts, int N, int K);
LSG_API int lsg_fp8_grouped_gemm(const lsg_fp8_grouped_gemm_params* p, int total_tokens, void* workspace,
                                 size_t workspace_bytes, void* stream);

/* bf16 weight [N,K] -> e4m3 [N,K] + one fp32 scale per 128 x 128 tile, stored K-major
 * (scales[kb + nb * ceil(K/128)]).  Not in-place safe. */
LSG_API int lsg_weight_fp8_quant(const void* weight_bf16, void* output_e4m3, float* scales, int N, int K,
                                 void* stream);

/* Mirrors struct DynamicFp8QuantParams, csrc/smxx/quant/dynamic_fp8_quant.h:25-32. */
typedef struct lsg_dynamic_fp8_quant_params {
    int num_tokens;     /* M */
    int hidden_size;    /* K */
    const void* input;  /* [M,K] bf16 */
    void* output;       /* [M,K] e4m3 bytes */
    void* scales;       /* fp32 [M,ceil(K/128)], or [ceil(K/128),M] when m_major_scales */
    int m_major_scales;
} lsg_dynamic_fp8_quant_params;

/* bf16 -> e4m3 with one fp32 scale per (token, 128-column block); bit-exact with the
 * reference.  Replaces launch_dynamic_fp8_quant,
 * csrc/smxx/quant/dynamic_fp8_quant.cu:118-147 (kernel :38-112). */
LSG_API int lsg_dynamic_fp8_quant(const lsg_dynamic_fp8_quant_params* p, void* stream);

/* Mirrors Bf16ToNvfp4GroupedParams (csrc/smxx/quant/bf16_to_nvfp4_grouped.h:15-33) and
 * SiluMulToNvfp4GroupedParams (silu_mul_to_nvfp4_grouped.h:15-35): `input` is the
 * activation, or the gate half when `up` is used. */
typedef struct lsg_nvfp4_grouped_quant_params {
    const void* input;          /* [T,K] bf16 (gate for the SwiGLU variant)          */
    const void* up;             /* [T,K] bf16, SwiGLU variant only                   */
    void* output_packed;        /* [T,K/2] e2m1 pairs, low nibble = even k           */
    void* output_scales;        /* ue4m3, interleaved 128x4 layout, per-expert       */
                                /* sections padded to 128 rows; caller zero-fills    */
    const void* expert_offsets; /* int32 [E+1], device                               */
    const void* sf_offsets;     /* int32 [E+1], device, in padded rows               */
    int total_tokens;
    int num_experts;
    int K;                      /* multiple of 16 (64 for the GEMM's scale atoms)    */
    const void* input_scales;   /* optional fp32 [E] per-expert global scales        */
} lsg_nvfp4_grouped_quant_params;

/* Replaces launch_bf16_to_nvfp4_grouped, csrc/smxx/quant/bf16_to_nvfp4_grouped.cu:99-113. */
LSG_API int lsg_bf16_to_nvfp4_grouped(const lsg_nvfp4_grouped_quant_params* p, void* stream);

/* Replaces launch_silu_mul_to_nvfp4_grouped,
 * csrc/smxx/quant/silu_mul_to_nvfp4_grouped.cu:121-139. */
LSG_API int lsg_silu_mul_to_nvfp4_grouped(const lsg_nvfp4_grouped_quant_params* p, void* stream);

/* sf_offsets[e] = rows of the experts before e, each rounded up to 128, on the device.
 * Replaces the host loop of the reference's binding, csrc/bindings_python.cu:312-326,
 * for callers that must not synchronize. */
LSG_API int lsg_nvfp4_sf_offsets(const int32_t* expert_offsets, int32_t* sf_offsets,
                                 int num_experts, void* stream);

/* ------------------------------------------------------------------------ */
/* NVFP4 grouped GEMM                                                       */
/* ------------------------------------------------------------------------ */

/* Mirrors struct Nvfp4GroupedGemmParams, csrc/sm120/gemm/grouped_gemm.h:34-57
 * (problem_sizes is accepted for interface parity; row counts come from expert_offsets). */
typedef struct lsg_nvfp4_grouped_gemm_params {
    int num_experts;
    int N;
    int K;
    const void* A_base;            /* [T,K/2] e2m1 pairs, low nibble = even k            */
    const void* B_base;            /* [E,N,K/2]                                          */
    void* D_base;                  /* [T,N] output_dtype                                 */
    const void* scale_A_base;      /* ue4m3, interleaved layout, sections per sf_offsets */
    const void* scale_B_base;      /* ue4m3, interleaved layout, N*K/16 bytes per expert */
    const float* alphas;           /* [E]                                                */
    const int32_t* expert_offsets; /* [E+1]                                              */
    const int32_t* sf_offsets;     /* [E+1] in padded rows                               */
    const int32_t* problem_sizes;  /* [E,3] {M_e,N,K}; may be null                       */
    int output_dtype;              /* LSG_DTYPE_BF16, _F16 (or _F32 as an extension)     */
    const void* const* B_ptrs;       /* optional [E] per-expert weight pointers          */
    const void* const* scale_B_ptrs; /* optional [E] per-expert scale pointers           */
} lsg_nvfp4_grouped_gemm_params;

/* Single-problem NVFP4 quantizer and GEMM.  Replace launch_bf16_to_nvfp4
 * (csrc/smxx/quant/bf16_to_nvfp4.cu:76-140), query_nvfp4_gemm_workspace_size and
 * launch_nvfp4_gemm (csrc/sm120/gemm/nvfp4/nvfp4_gemm.cu:189-200).  Scale buffers use the
 * interleaved layout of lsg_nvfp4_sf_buffer_bytes(rows, K); the quantizer does not write the
 * padding entries (callers zero the buffer first, as the reference's binding does).  The GEMM
 * takes the block-scaled tensor-core instruction when K is a multiple of 64 and the four
 * buffers are 16-byte aligned (no workspace is touched then), else the fp16 expansion. */
LSG_API int lsg_bf16_to_nvfp4(const void* x_bf16, void* output_packed, void* output_scales, int M, int K,
                              void* stream);
/* NVFP4 weight -> bf16: codes [N, K/2], RAW row-major ue4m3 group scales [N, K/16] (not the
 * interleaved layout), global scalar; out[n,k] = (e2m1 * scale) * weight_scale_2 rounded to
 * bf16.  Replaces launch_nvfp4_dequant_bf16, csrc/smxx/quant/nvfp4_dequant_bf16.cu:86-121. */
LSG_API int lsg_nvfp4_dequant_bf16(const void* input_packed, const void* scales, float weight_scale_2,
                                   void* output_bf16, int N, int K, void* stream);
typedef struct lsg_nvfp4_gemm_params {
    int M, N, K;
    const void* A;        /* [M, K/2] e2m1 codes, low nibble = even k   */
    const void* B;        /* [N, K/2]                                   */
    void* D;              /* [M, N] output_dtype                        */
    const void* scale_A;  /* ue4m3, interleaved layout of (M, K/16)     */
    const void* scale_B;  /* ue4m3, interleaved layout of (N, K/16)     */
    float alpha;          /* output scale                               */
    int output_dtype;     /* LSG_DTYPE_BF16, _F16 or _F32               */
} lsg_nvfp4_gemm_params;
LSG_API size_t lsg_nvfp4_gemm_workspace_bytes(int M, int N, int K);
LSG_API int lsg_nvfp4_gemm(const lsg_nvfp4_gemm_params* p, void* workspace, size_t workspace_bytes,
                           void* stream);

/* Replaces query_nvfp4_grouped_gemm_workspace_size (nvfp4_grouped_gemm.cu:373-384).  The
 * operator runs on tcgen05.mma.kind::mxf4nvf4.block_scale straight from the caller's packed
 * buffers and then needs only the token-tile map (a few KB).  Calls that cannot take that
 * route - weight pointer arrays (B_ptrs / scale_B_ptrs), K not a multiple of 64, operands or
 * scale buffers that are not 16-byte aligned - expand both operands to fp16 in the workspace
 * and need the `_ex(..., 1)` size (total_tokens*K*2 + num_experts*N*K*2 bytes more). */
LSG_API size_t lsg_nvfp4_grouped_gemm_workspace_bytes(int total_tokens, int num_experts, int N, int K);
LSG_API size_t lsg_nvfp4_grouped_gemm_workspace_bytes_ex(int total_tokens, int num_experts, int N, int K,
                                                         int expanded);

/* Replaces launch_nvfp4_grouped_gemm, nvfp4_grouped_gemm.cu:386-423.  Device-routed (no
 * host synchronization); rows of empty experts are left untouched. */
LSG_API int lsg_nvfp4_grouped_gemm(const lsg_nvfp4_grouped_gemm_params* p, int total_tokens,
                                   void* workspace, size_t workspace_bytes, void* stream);

/* fp32 scales [rows, K/16] -> ue4m3 in the interleaved layout (rows padded to 128, groups
 * to 4; dst must hold lsg_nvfp4_sf_buffer_bytes(rows, K) zero-filled bytes).
 * Replaces launch_reformat_scales, csrc/smxx/quant/reformat_scales.cu:63-69, and
 * query_sf_buffer_size_b. */
LSG_API size_t lsg_nvfp4_sf_buffer_bytes(int rows, int K);
LSG_API int lsg_nvfp4_reformat_scales(const float* src, void* dst, int rows, int K, void* stream);

/* ------------------------------------------------------------------------ */
/* MoE routing, permutation, combine                                        */
/* No counterpart in the reference: its grouped operators take rows that are */
/* already grouped by expert (gguf_grouped_gemm.h:20-24).                   */
/* ------------------------------------------------------------------------ */

/* p = softmax(logits fp32 [T,E]); top-k (ties to the lower expert id); weights renormalised
 * to sum 1.  topk_idx int32 [T,k], topk_weights fp32 [T,k].  E <= 1024, k <= 16. */
LSG_API int lsg_moe_route(const float* logits, int num_tokens, int num_experts, int top_k,
                          int32_t* topk_idx, float* topk_weights, void* stream);

/* Stable grouping of the T*k (token, slot) pairs by expert: expert_offsets int32 [E+1],
 * perm int32 [T*k] (row -> pair), inv_perm int32 [T*k] (pair -> row).
 * E <= 1024.  Pairs with an expert id outside [0, E) get no row.
 * counts_scratch: int32 [lsg_moe_permutation_scratch_ints(T, k, E)] (per-chunk histograms
 * of a counting sort over chunks of 256 pairs). */
LSG_API long long lsg_moe_permutation_scratch_ints(int num_tokens, int top_k, int num_experts);
LSG_API int lsg_moe_permutation(const int32_t* topk_idx, int num_tokens, int top_k, int num_experts,
                                int32_t* expert_offsets, int32_t* perm, int32_t* inv_perm,
                                int32_t* counts_scratch, void* stream);

/* Expert-parallel receive side.  After the all-to-all a rank holds `rows` rows grouped by
 * (source rank, local expert); recv_counts int32 [world * experts_per_rank] gives the block
 * sizes in that order.  Writes local_offsets int32 [experts_per_rank + 1] (rows per local
 * expert, cumulative), order int32 [rows] (destination row -> received row, destination =
 * grouped by (local expert, source rank)) and its inverse.  scratch: int32
 * [2 * world * experts_per_rank].  world * experts_per_rank <= 1024.  Rows whose blocks have
 * size zero do not exist; an empty-before-i search keeps the order stable.  No counterpart in
 * the reference (it has no multi-GPU code). */
LSG_API int lsg_ep_expert_order(const int32_t* recv_counts, int world, int experts_per_rank, int rows,
                                int32_t* local_offsets, int32_t* order, int32_t* inv_order,
                                int32_t* scratch, void* stream);

/* Expert-parallel exchange over peer memory (one node, one process per GPU, NVLink): the
 * routed rows are stored straight into the destination GPU's receive buffer and the expert
 * outputs straight back into the sender's return buffer, by plain kernels; no all-to-all
 * collective, no host round trip.  Rank r owns experts [r*E/world, (r+1)*E/world).
 * The `*_ptrs` arguments are DEVICE arrays of `world` device pointers, entry p = rank p's
 * buffer (entry `rank` = the local one); the buffers must be peer-accessible (symmetric
 * allocations).  The caller separates the steps with a barrier over all ranks on the stream:
 *   publish_counts | barrier | plan, send_rows | barrier | (expert block) | return_rows | barrier
 * counts table: int32 [world][E]; receive buffer: bf16 [capacity][H], rows grouped by
 * (local expert, source rank), described by local_offsets int32 [E/world + 1]; return buffer:
 * bf16 [num_pairs][H] in the sender's sorted-by-expert order.  send_base int32 [E], dst_start
 * and ret_base int32 [E] (world * E/world), info int32 [2] = {rows received, overflow flag};
 * E <= 1024, H % 8 == 0.
 * Overflow: when the ranks send a rank more rows than its `capacity`, lsg_ep_plan clamps every
 * start and offset it writes (local_offsets, dst_start, info[0]) to `capacity`, sets info[1]
 * on every rank and records code 7 in the device status word (lsg_device_status);
 * lsg_ep_send_rows drops the rows that do not fit and clears their slots of `back_local`
 * (this rank's own return buffer, may be NULL), so a dropped row contributes zeros to the
 * combine instead of the previous layer's output.  Nothing is written past `capacity`.
 * No counterpart in the reference (it has no multi-GPU code). */
LSG_API int lsg_ep_publish_counts(const int32_t* expert_offsets, int num_experts, int rank, int world,
                                  void* const* counts_table_ptrs, void* stream);
LSG_API int lsg_ep_plan(const int32_t* counts_table, int rank, int world, int num_experts, int capacity,
                        int32_t* send_base, int32_t* local_offsets, int32_t* dst_start, int32_t* ret_base,
                        int32_t* info, void* stream);
LSG_API int lsg_ep_send_rows(const void* hidden_bf16, const int32_t* perm, const int32_t* expert_offsets,
                             const int32_t* send_base, int num_pairs, int top_k, int H, int num_experts, int world,
                             void* const* recv_buf_ptrs, int capacity, void* back_local, void* stream);
LSG_API int lsg_ep_return_rows(const void* y_bf16, const int32_t* dst_start, const int32_t* ret_base,
                               const int32_t* info, int world, int experts_per_rank, int H, int capacity,
                               void* const* back_buf_ptrs, void* stream);
/* The same two steps for one group of each rank's local experts, [local_expert_lo, local_expert_hi)
 * in the rank-local numbering: send_rows_group sends only the rows routed to those experts of
 * every rank (they are contiguous in the receive layout, rows local_offsets[lo] ..
 * local_offsets[hi]), return_rows_group returns only those rows of `y_bf16` (local_offsets as
 * written by lsg_ep_plan).  A caller can then exchange one group's rows while the expert GEMMs
 * of another group run on a second stream (distributed.EpPeerGroups); each group's steps need
 * their own barrier flags.  No counterpart in the reference. */
LSG_API int lsg_ep_send_rows_group(const void* hidden_bf16, const int32_t* perm, const int32_t* expert_offsets,
                                   const int32_t* send_base, int num_pairs, int top_k, int H, int num_experts,
                                   int world, void* const* recv_buf_ptrs, int capacity, void* back_local,
                                   int local_expert_lo, int local_expert_hi, void* stream);
LSG_API int lsg_ep_return_rows_group(const void* y_bf16, const int32_t* dst_start, const int32_t* ret_base,
                                     const int32_t* info, int world, int experts_per_rank, int H, int capacity,
                                     void* const* back_buf_ptrs, const int32_t* local_offsets, int local_expert_lo,
                                     int local_expert_hi, void* stream);

/* Barrier over the ranks of the exchange, on the stream, with a time limit.  flag_ptrs is a
 * DEVICE array of `world` device pointers, entry p = rank p's flag array uint32 [world + 1]
 * in peer-accessible memory, zeroed once before the first use (all ranks zero, then
 * synchronize once on the host).  mode 3 = arrive and wait (the normal call); 1 = arrive only,
 * 2 = wait only (tests that emulate several ranks on one GPU).  A rank whose peers do not
 * arrive within the wait limit (lsg_set_wait_limit_cycles) records code 6 in the device status
 * word and returns; nothing waits without a limit and no multicast is used.  world <= 64.
 * No counterpart in the reference. */
LSG_API int lsg_ep_barrier(void* const* flag_ptrs, int rank, int world, int mode, void* stream);

/* out[row,:] = hidden[perm[row] / top_k, :]   (bf16, H multiple of 8). */
LSG_API int lsg_moe_permute(const void* hidden_bf16, const int32_t* perm, int rows, int top_k, int H,
                            void* out_bf16, void* stream);

/* out[t,:] = sum over slots s (in order) of topk_weights[t,s] * y[inv_perm[t*k+s], :],
 * fp32 fused multiply-adds, rounded to bf16. */
LSG_API int lsg_moe_unpermute(const void* y_bf16, const int32_t* inv_perm, const float* topk_weights,
                              int num_tokens, int top_k, int H, void* out_bf16, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LSG_H_ */
