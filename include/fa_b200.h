/*
 * C ABI of the B200 (sm_100a) flash-attention forward library, libfa_b200.so.
 *
 * This is the boundary a foreign-function binding attaches to: plain pointers,
 * sizes and ints, no C++ or framework types.  Every entry point returns FA_OK
 * (0) or a negative FA_ERR_* code and never terminates the process.
 *
 * The C++ interface of the reference project stays available, source
 * compatible, in include/flash_attention.h (transformer::FlashAttentionParams,
 * transformer::launch_flash_attention); it is a thin shim over fa_prefill().
 *
 * Tensors are dense, row-major, [batch_size * num_heads, seq_len, d_head],
 * exactly the layout the reference documents (include/flash_attention.h:21-22,
 * 52-56).  LSE is the natural-log log-sum-exp of the scaled scores, fp32,
 * [batch_size * num_heads, seq_len] (kernels/flash_attention.cu:498-505).
 * Causal masking keeps key j for query i iff j <= i
 * (kernels/flash_attention.cu:307-312, oracle src/demo.cu:41).
 *
 * All device pointers must be 16-byte aligned.  Kernels are enqueued on the
 * given stream and the call returns without synchronising, like the
 * reference's launch (kernels/flash_attention.cu:567-578).
 */
#ifndef FA_B200_H_
#define FA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FA_OK                    0
#define FA_ERR_INVALID_ARGUMENT (-1)  /* null pointer, non-positive size, scale <= 0 or not finite */
#define FA_ERR_UNSUPPORTED      (-2)  /* d_head / dtype / split count outside what is built */
#define FA_ERR_MISALIGNED       (-3)  /* a device pointer is not 16-byte aligned */
#define FA_ERR_WORKSPACE        (-4)  /* workspace missing or too small */
#define FA_ERR_CUDA             (-5)  /* a CUDA runtime/driver call failed; see fa_last_cuda_error() */
#define FA_ERR_DEVICE_TIMEOUT   (-6)  /* a kernel gave up on a bounded wait; see fa_device_status() */
#define FA_ERR_NOT_SM100        (-7)  /* the current device is not compute capability 10.x */
#define FA_ERR_NCCL             (-8)  /* an NCCL call failed, or libnccl.so.2 could not be loaded */

enum { FA_DTYPE_F16 = 0, FA_DTYPE_BF16 = 1, FA_DTYPE_E4M3 = 2 };

/*
 * Prefill (self-attention forward, Sq == Skv).  Replaces
 * transformer::launch_flash_attention (include/flash_attention.h:51-67,
 * kernels/flash_attention.cu:595-617) and the kernel behind it
 * (kernels/flash_attention.cu:116-507).
 *
 * dtype F16 : q,k,v,o fp16.        dtype BF16: q,k,v,o bf16.
 * dtype E4M3: q,k,v e4m3 codes with per-(batch*head) dequantisation scales
 *             q_scale,k_scale,v_scale (device, fp32, [batch_size*num_heads],
 *             value = code * scale); o bf16.
 *             The call first writes an fp16 copy of v (P V runs on the 16-bit
 *             tensor-core kind) into scratch memory that it takes, in stream
 *             order, from a memory pool of the library's own and returns the same
 *             way (cudaMallocFromPoolAsync / cudaFreeAsync on args->stream): at
 *             most 256 MB, heads processed in chunks beyond that; the pool keeps
 *             the memory, so only the first call per device allocates.
 * d_head 64 or 128 (E4M3: 128 only).  seq_len any positive value.
 */
typedef struct fa_prefill_args {
    const void*  q;
    const void*  k;
    const void*  v;
    void*        o;
    float*       lse;          /* optional, may be NULL */
    int          batch_size;
    int          num_heads;
    int          seq_len;
    int          d_head;
    float        scale;        /* > 0, typically 1/sqrt(d_head) */
    int          causal;       /* 0 / 1 */
    int          dtype;        /* FA_DTYPE_* */
    const float* q_scale;      /* E4M3 only, else NULL */
    const float* k_scale;
    const float* v_scale;
    void*        stream;       /* cudaStream_t */
} fa_prefill_args;

int fa_prefill(const fa_prefill_args* args);

/*
 * fa_prefill has two kernels for 16-bit inputs, as the reference has two tile variants
 * behind its dispatcher (kernels/flash_attention.cu:595-617: 32x64 tiles while
 * B*H*ceil(S/64) < 2 * SMs, else 64x64).  FA_PREFILL_ONE_TILE walks one 128-row query tile
 * per CTA with two softmax groups on alternate key tiles; FA_PREFILL_TILE_PAIR walks two
 * query tiles per CTA, each K/V tile in shared memory feeding both (half the K/V traffic
 * from L2).  FA_PREFILL_AUTO (the default) picks the one measured faster, today the one-tile
 * kernel on every shape.  This call overrides the choice for the whole process (tests and
 * tuning).  Results are the same within the stated tolerances.
 */
enum { FA_PREFILL_AUTO = 0, FA_PREFILL_ONE_TILE = 1, FA_PREFILL_TILE_PAIR = 2, FA_PREFILL_CTA_PAIR = 3 };
int fa_set_prefill_variant(int variant);

/*
 * Same computation with HOST buffers: copies q,k,v (and the scales) to the
 * device, runs fa_prefill, copies o (and lse) back and synchronises.  This is
 * the call pattern of the reference's own verification and demo programs
 * (src/bench.cu:250-275, src/demo.cu:282-322: cudaMalloc, cudaMemcpy H2D,
 * launch, cudaMemcpy D2H) folded into one entry point.  Device staging
 * buffers are kept per device and grown on demand.  Large inputs are cut into
 * chunks of heads that flow through three internal streams, so the copies in
 * both PCIe directions and the kernels overlap; use pinned host memory to
 * benefit.  `stream` is ignored.  Calls on the same device are serialised inside the
 * library (they share the staging buffers and streams); calls on different devices run
 * concurrently.
 */
int fa_prefill_host(const fa_prefill_args* args_with_host_pointers);

/*
 * Split-KV decode: one query row per (batch, head) against a KV cache of
 * seq_len_kv keys, every key visible (no mask).  The reference has no decode
 * path; the definition is the reference attention (src/demo.cu:28-70) applied
 * to a single query row.  q, o: [batch_size*num_heads, d_head]; k, v:
 * [batch_size*num_heads, seq_len_kv, d_head]; fp16 or bf16; d_head 64 or 128.
 *
 * The key range is cut into num_splits contiguous slices (0 = choose); each
 * slice produces a partial (O, LSE) in `workspace`, and a second kernel merges
 * the partials by their LSEs and writes o (16-bit) and, if given, lse.
 * If o_f32 is non-NULL the merged, normalised output is ALSO written there in
 * fp32 ([batch_size*num_heads, d_head]); together with lse this is the partial
 * result a rank contributes when the KV sequence is sharded across GPUs.
 */
typedef struct fa_decode_args {
    const void* q;
    const void* k;
    const void* v;
    void*       o;             /* may be NULL when o_f32 is given */
    float*      lse;           /* optional unless o_f32 is given */
    float*      o_f32;         /* optional */
    int         batch_size;
    int         num_heads;
    int         seq_len_kv;
    int         d_head;
    float       scale;
    int         dtype;         /* FA_DTYPE_F16 or FA_DTYPE_BF16 */
    int         num_splits;    /* 0 = library chooses; else 1..FA_MAX_SPLITS */
    void*       workspace;     /* device, >= fa_decode_workspace_bytes(...) */
    size_t      workspace_bytes;
    void*       stream;
} fa_decode_args;

#define FA_MAX_SPLITS 256

size_t fa_decode_workspace_bytes(int batch_size, int num_heads, int d_head, int num_splits);
int    fa_decode_default_splits(int batch_size, int num_heads, int seq_len_kv);
int    fa_decode(const fa_decode_args* args);

/*
 * fa_decode without any allocation on either side.  (No counterpart in the
 * reference, which has no decode path and allocates nothing per call.)
 *
 * Who needs it: hosts that hand the whole device to their own memory pool at
 * start-up and forbid cudaMalloc afterwards (a serving runtime with a frozen
 * arena, a plugin sandbox, a latency-critical loop where the device-wide
 * synchronisation implied by cudaMalloc/cudaFree is not acceptable).  Such a
 * caller cannot size and allocate the split-KV workspace fa_decode asks for.
 *
 * Here the per-split partial results live in an array built into the library
 * image (FA_DECODE_STATIC_SCRATCH_BYTES of device memory, held by every GPU
 * that loads the library until the process exits).  The caller passes inputs
 * and outputs exactly as for fa_decode; `workspace` and `workspace_bytes` are
 * ignored.  The call allocates nothing: no cudaMalloc, no cudaFree, no
 * allocating library routine.
 *
 * Limit: batch_size*num_heads*splits*(d_head+1)*4 bytes (each part rounded up
 * to 256) must fit in FA_DECODE_STATIC_SCRATCH_BYTES; beyond that the call
 * launches nothing and returns FA_ERR_WORKSPACE.  Lower num_splits to fit.
 *
 * The first call on each device looks up the array's device address (once,
 * with that device current); make that first call during start-up and before
 * starting any stream capture: with CUDA's lazy module loading that lookup can
 * be the moment the driver loads this library's device code and backs the
 * array with memory, which is the driver's allocation, not the library's, and
 * happens once.  Every later call only launches kernels.  All calls on a device share the one array: it still holds the
 * previous call's partials (every slot a call reads is first written by that
 * call, so nothing needs clearing), and two calls whose kernels overlap on the
 * GPU - different streams, or different host threads - race on it.  Serialise
 * them, or use fa_decode with separate workspaces.
 */
#define FA_DECODE_STATIC_SCRATCH_BYTES (8u * 1024u * 1024u + 512u * 1024u)
int fa_decode_static(const fa_decode_args* args);

/* ---------------------------------------------------------------------------
 * fa_decode_gqa: grouped-query / multi-query decode over a strided KV cache.
 * No reference counterpart (the reference has one K/V head per query head and
 * dense tensors, include/flash_attention.h:46-61); the result is defined as
 * cpu_attention (src/demo.cu:28-70) applied per query head hq, one query row,
 * with K and V of KV head hq / (num_q_heads / num_kv_heads).
 *
 *   q   [B, Hq, D] dense;  o [B, Hq, D];  lse [B, Hq] (optional, natural log)
 *   k,v key r of KV head h of sequence b at element offset
 *           b * kv_batch_stride + h * kv_head_stride + r * kv_row_stride
 *       (rows of D contiguous elements; the three strides multiples of 8 elements;
 *        all zero = dense [B, Hkv, Skv, D]).  A cache laid out [B, Skv, Hkv, D] is
 *        kv_row_stride = Hkv*D, kv_head_stride = D, kv_batch_stride = Skv*Hkv*D.
 *
 *   Paged cache (block_table != NULL): k and v point at pools of pages of
 *       page_size keys (a power of two >= 16); key r of KV head h of sequence b
 *       lives in page p = block_table[b * block_table_stride + r / page_size] at
 *           p * kv_page_stride + (r % page_size) * kv_row_stride + h * kv_head_stride
 *       (kv_batch_stride is ignored; num_pages is the size of the pool).
 *   seq_lens (optional, device, [B]): KV length of each sequence, clamped to
 *       [0, seq_len_kv]; seq_len_kv then is the maximum and sizes the splits.  A
 *       sequence of length 0 yields O = 0 and LSE = -inf.  Cache contents past a
 *       sequence's end are never used (they may be uninitialised).
 *
 *   dtype FA_DTYPE_E4M3 (d_head 128 only): q, k and v hold e4m3 codes, the value of an
 *       element of sequence b, KV head h being code * {q,k,v}_scale[b * num_kv_heads + h]
 *       (device arrays of B * num_kv_heads floats; the query heads of a group share the
 *       scale); o is bf16; strides are multiples of 16 elements.  Q K^T runs on the 8-bit
 *       tensor-core kind, V is converted to fp16 in shared memory (exact), P is fp16: the
 *       cache is read at one byte per element.
 *
 *   num_q_tokens = T > 1 (speculative / multi-token decode, appended chunks): q and o are
 *       [B, T, Hq, D], lse [B, T, Hq]; the T tokens are the last T entries of each sequence's
 *       cache and token t sees keys [0, len - T + t] (any T: 128 / group tokens share a query
 *       tile, so a long T is a prefill chunk appended to a cached prefix); the workspace is
 *       fa_decode_workspace_bytes(B, T * Hq, D, splits), and with num_splits = 0 the library
 *       uses fa_decode_gqa_default_splits(B * ceil(T / (128 / group)), Hkv, Skv).  A token of a
 *       sequence shorter than T that sees no key yields O = 0, LSE = -inf.
 *
 * The group of num_q_heads / num_kv_heads (<= 128) query heads that share a KV
 * head occupies the rows of one tensor-core query tile, so K and V stream from
 * HBM once per KV head whatever the group size.  The KV length is split over
 * CTAs; partial results go through `workspace`
 * (>= fa_decode_workspace_bytes(B, Hq, D, splits) with
 * splits = num_splits, or fa_decode_gqa_default_splits(...) when num_splits is 0)
 * and are merged by the combine kernel.
 * ------------------------------------------------------------------------- */
typedef struct fa_decode_gqa_args {
    const void* q;
    const void* k;
    const void* v;
    void*       o;
    float*      lse;              /* optional */
    int         batch_size;
    int         num_q_heads;
    int         num_kv_heads;     /* divides num_q_heads */
    int         seq_len_kv;
    int         d_head;           /* 64 or 128 */
    float       scale;
    int         dtype;            /* FA_DTYPE_F16, FA_DTYPE_BF16 or FA_DTYPE_E4M3 */
    int         num_splits;       /* 0 = library chooses; else 1..FA_MAX_SPLITS */
    long long   kv_batch_stride;  /* elements; see above */
    long long   kv_head_stride;
    long long   kv_row_stride;
    const int*  block_table;      /* device; NULL = not paged */
    int         block_table_stride;
    int         page_size;
    int         num_pages;
    long long   kv_page_stride;
    const int*  seq_lens;         /* device; NULL = every sequence has seq_len_kv keys */
    const float* q_scale;         /* e4m3 only */
    const float* k_scale;
    const float* v_scale;
    int         num_q_tokens;     /* 0 or 1 = one query token per sequence */
    void*       workspace;
    size_t      workspace_bytes;
    void*       stream;
} fa_decode_gqa_args;

int fa_decode_gqa_default_splits(int batch_size, int num_kv_heads, int seq_len_kv);
int fa_decode_gqa(const fa_decode_gqa_args* args);

/* ---------------------------------------------------------------------------
 * fa_backward: dQ, dK, dV of the prefill forward.  No reference counterpart (the
 * reference is forward only; its kernel stores L "for the backward pass",
 * kernels/flash_attention.cu:497).  Definition: the gradient of
 * O = softmax(scale * Q K^T [causal mask]) V (src/demo.cu:28-70) with respect to
 * Q, K, V for an upstream gradient dO, using the forward's O and LSE:
 *     P = exp(scale * Q K^T - LSE), dV = P^T dO, dS = P o (dO V^T - delta) * scale,
 *     delta_i = sum_d dO_id O_id, dQ = dS K, dK = dS^T Q.
 * All tensors dense [B*H, S, D] in `dtype` (f16 or bf16), lse fp32 [B*H, S]
 * (natural log, as fa_prefill writes it); d_head 64 or 128.  workspace:
 * fa_backward_workspace_bytes(B, H, S) bytes of device memory (fp32 delta).
 * ------------------------------------------------------------------------- */
typedef struct fa_backward_args {
    const void*  q;
    const void*  k;
    const void*  v;
    const void*  o;           /* forward output */
    const void*  d_o;         /* upstream gradient, same layout as o */
    const float* lse;         /* forward log-sum-exp */
    void*        dq;
    void*        dk;
    void*        dv;
    int          batch_size;
    int          num_heads;
    int          seq_len;
    int          d_head;
    float        scale;
    int          causal;
    int          dtype;
    void*        workspace;
    size_t       workspace_bytes;
    void*        stream;
} fa_backward_args;

size_t fa_backward_workspace_bytes(int batch_size, int num_heads, int seq_len);
int fa_backward(const fa_backward_args* args);

/*
 * LSE merge of n_parts partial results (the exchange step of KV-sequence
 * sharded decode: each rank's (o_f32, lse) gathered into one local buffer).
 *   o_parts  : fp32 [n_parts, rows, d_head]   lse_parts: fp32 [n_parts, rows]
 *   o        : 16-bit [rows, d_head] (dtype F16 or BF16)   lse: optional [rows]
 * m = max_p lse_p; w_p = exp(lse_p - m); o = sum w_p o_p / sum w_p;
 * lse = m + log(sum w_p).
 */
int fa_combine(const float* o_parts, const float* lse_parts, int n_parts, int rows, int d_head,
               void* o, float* lse, int dtype, void* stream);

/*
 * The same merge over PACKED partials: packed_parts is fp32 [n_parts, rows, d_head + 1], a row
 * holding the normalised partial O followed by its LSE - exactly the receive buffer of one
 * all-gather of every rank's [rows, d_head + 1] block, read where it lies (no unpacking pass).
 */
int fa_combine_packed(const float* packed_parts, int n_parts, int rows, int d_head, void* o,
                      float* lse, int dtype, void* stream);

/*
 * KV-sequence-sharded decode, the one multi-GPU path with an exchange step (the reference is
 * single-GPU; the definition is src/demo.cu:28-70 on the whole cache, which the LSE merge of
 * per-slice results reproduces).  Every rank holds a contiguous slice of the keys of ALL heads
 * and calls this with the same batch_size / num_heads / d_head / dtype:
 *     1. split-KV decode on the local slice (args->k, args->v, args->seq_len_kv = local keys;
 *        0 is allowed: the rank then contributes weight zero), whose merge writes this rank's
 *        packed [rows, d_head + 1] block straight into its place in `gather`;
 *     2. ONE ncclAllGather, in place, of that block (rows * (d_head + 1) floats per rank);
 *     3. fa_combine_packed over the gathered blocks -> args->o (16-bit) and args->lse, the
 *        same on every rank.
 * All on args->stream: partial kernel, merge kernel, all-gather, merge kernel (4 launches).
 * nccl_comm is the caller's ncclComm_t (one rank per GPU); gather is device memory of
 * fa_decode_kv_sharded_gather_bytes(...) bytes, reusable across calls; args->workspace as
 * for fa_decode; args->o_f32 is ignored.  NCCL is loaded at run time (libnccl.so.2 - the
 * copy already in the process, if any), the library does not link against it.
 *
 * fa_nccl_unique_id / fa_nccl_comm_create / fa_nccl_comm_destroy forward to
 * ncclGetUniqueId / ncclCommInitRank / ncclCommDestroy of that same NCCL, for bindings
 * that cannot include <nccl.h> (the id is 128 bytes; rank 0 creates it and hands it to the
 * others by any side channel).
 */
size_t fa_decode_kv_sharded_gather_bytes(int batch_size, int num_heads, int d_head, int n_ranks);
int    fa_decode_kv_sharded(const fa_decode_args* args, void* nccl_comm, float* gather, size_t gather_bytes);
int    fa_nccl_unique_id(void* id_out, size_t id_bytes);
int    fa_nccl_comm_create(void** comm_out, int n_ranks, const void* id, size_t id_bytes, int rank);
int    fa_nccl_comm_destroy(void* comm);

/*
 * Tensor-core known-answer test (the role of test_ptx_mma in the reference,
 * src/bench.cu:51-165, for the tcgen05 path): one CTA computes
 *   S = Q K^T            (Q [128,d_head], K [128,d_head], 16-bit, from host)
 *   P = round16(S * p_scale)
 *   O = P V              (V [128,d_head])
 * through the same TMA tensor maps, shared-memory descriptors, TMEM layout and
 * instruction descriptors the attention kernels use, and returns S [128,128]
 * and O [128,d_head] in fp32 to host memory.  Synchronous.
 */
int fa_kat(int dtype, int d_head, const void* q_host, const void* k_host, const void* v_host,
           float p_scale, float* s_out_host, float* o_out_host);

/*
 * Device status word of the current device: 0, or the first error a kernel
 * recorded since the last clear ((code << 16) | detail; code 1 = a bounded
 * wait timed out, detail = barrier id).  Synchronises the device.
 */
int         fa_device_status(int* status_word);
/* The return code fa_device_status / fa_prefill_host derive from a status word (no device access). */
int         fa_status_word_to_error(int status_word);
int         fa_clear_device_status(void);
const char* fa_error_string(int code);
const char* fa_last_cuda_error(void);
int         fa_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FA_B200_H_ */
