// Entry points of libfa_b200.so that do not own a kernel: argument validation
// and dispatch for prefill, the host-buffer convenience call, device status,
// and the C++ shim transformer::launch_flash_attention that keeps the reference
// project's launch interface (include/flash_attention.h:51-67) working.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/flash_attention.h"
#include "bounded_wait.h"
#include "host_common.h"

namespace fa {

namespace {
constexpr int kMaxDevices = 64;
DeviceState g_states[kMaxDevices];
std::mutex  g_mutex;
thread_local char g_last_cuda_error[256] = "";

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
}  // namespace

int note_cuda_error(cudaError_t err, const char* where) {
    snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s: %s", where, cudaGetErrorString(err));
    return FA_ERR_CUDA;
}
int note_message(const char* msg, int code) {
    snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s", msg);
    return code;
}
int note_driver_error(CUresult err, const char* where) {
    snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s: CUresult %d", where, (int)err);
    return FA_ERR_CUDA;
}

DeviceState* device_state() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    DeviceState* st = &g_states[dev];
    // `ready` is release-stored after the fields and acquire-loaded before them, so a thread that
    // sees it set also sees the fields (several host threads may make the first call at once)
    if (st->ready.load(std::memory_order_acquire)) return st;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (st->ready.load(std::memory_order_relaxed)) return st;
    int sms = 0, major = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return nullptr;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return nullptr;
    int* status = nullptr;
    if (cudaMalloc(&status, sizeof(int)) != cudaSuccess) return nullptr;
    if (cudaMemset(status, 0, sizeof(int)) != cudaSuccess) return nullptr;
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess || !fn)
            return nullptr;
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    st->sm_count = sms;
    st->cc_major = major;
    st->status   = status;
    st->device   = dev;
    st->ready.store(true, std::memory_order_release);
    return st;
}

int make_tensor_map_3d(CUtensorMap* out, const void* base, int dtype, uint64_t row_elems,
                       uint64_t n_rows, uint64_t n_heads, uint32_t box_cols, uint32_t box_rows) {
    const uint64_t es = (dtype == FA_DTYPE_E4M3) ? 1 : 2;
    const CUtensorMapDataType dt = (dtype == FA_DTYPE_E4M3)   ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                   : (dtype == FA_DTYPE_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                              : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    cuuint64_t dims[3]    = {row_elems, n_rows, n_heads};
    cuuint64_t strides[2] = {row_elems * es, row_elems * n_rows * es};
    cuuint32_t box[3]     = {box_cols, box_rows, 1};
    cuuint32_t estr[3]    = {1, 1, 1};
    CUresult r = g_encode(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return note_driver_error(r, "cuTensorMapEncodeTiled");
    return FA_OK;
}

int make_tensor_map_4d(CUtensorMap* out, const void* base, int dtype, uint64_t row_elems,
                       uint64_t n_rows, uint64_t n_heads, uint64_t n_blocks, uint64_t row_stride,
                       uint64_t head_stride, uint64_t block_stride, uint32_t box_cols, uint32_t box_rows) {
    const uint64_t es = (dtype == FA_DTYPE_E4M3) ? 1 : 2;
    const CUtensorMapDataType dt = (dtype == FA_DTYPE_E4M3)   ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                   : (dtype == FA_DTYPE_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                              : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    cuuint64_t dims[4]    = {row_elems, n_rows, n_heads, n_blocks};
    cuuint64_t strides[3] = {row_stride * es, head_stride * es, block_stride * es};
    cuuint32_t box[4]     = {box_cols, box_rows, 1, 1};
    cuuint32_t estr[4]    = {1, 1, 1, 1};
    CUresult r = g_encode(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return note_driver_error(r, "cuTensorMapEncodeTiled");
    return FA_OK;
}

int make_tensor_map_q5(CUtensorMap* out, const void* base, int dtype, uint64_t d_head, uint64_t group,
                       uint64_t n_tok, uint64_t n_kv_heads, uint64_t batch, uint32_t box_cols) {
    const uint64_t es = (dtype == FA_DTYPE_E4M3) ? 1 : 2;
    const CUtensorMapDataType dt = (dtype == FA_DTYPE_E4M3)   ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                   : (dtype == FA_DTYPE_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                              : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const uint64_t hq = group * n_kv_heads;
    cuuint64_t dims[5]    = {d_head, group, n_tok, n_kv_heads, batch};
    cuuint64_t strides[4] = {d_head * es, hq * d_head * es, group * d_head * es, n_tok * hq * d_head * es};
    const uint64_t per_tile = 128 / group < n_tok ? 128 / group : n_tok;     // tokens per query tile
    cuuint32_t box[5]     = {box_cols, (cuuint32_t)group, (cuuint32_t)per_tile, 1, 1};
    cuuint32_t estr[5]    = {1, 1, 1, 1, 1};
    CUresult r = g_encode(out, dt, 5, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return note_driver_error(r, "cuTensorMapEncodeTiled");
    return FA_OK;
}

namespace {

int validate_prefill(const fa_prefill_args* a) {
    if (!a || !a->q || !a->k || !a->v || !a->o) return FA_ERR_INVALID_ARGUMENT;
    if (a->batch_size <= 0 || a->num_heads <= 0 || a->seq_len <= 0) return FA_ERR_INVALID_ARGUMENT;
    if (!(a->scale > 0.0f) || !std::isfinite(a->scale)) return FA_ERR_INVALID_ARGUMENT;
    if ((long long)a->batch_size * a->num_heads > 0x7FFFFFFFll) return FA_ERR_INVALID_ARGUMENT;
    if (a->dtype != FA_DTYPE_F16 && a->dtype != FA_DTYPE_BF16 && a->dtype != FA_DTYPE_E4M3)
        return FA_ERR_UNSUPPORTED;
    if (a->d_head != 64 && a->d_head != 128) return FA_ERR_UNSUPPORTED;
    if (a->dtype == FA_DTYPE_E4M3) {
        if (a->d_head != 128) return FA_ERR_UNSUPPORTED;
        if (!a->q_scale || !a->k_scale || !a->v_scale) return FA_ERR_INVALID_ARGUMENT;
    }
    return FA_OK;
}

// Grows staging buffer `slot` of the current device to at least `bytes`.
int stage_reserve(DeviceState* st, int slot, size_t bytes) {
    if (st->stage_bytes[slot] >= bytes) return FA_OK;
    if (st->stage[slot]) FA_CUDA_TRY(cudaFree(st->stage[slot]));
    st->stage[slot] = nullptr;
    st->stage_bytes[slot] = 0;
    FA_CUDA_TRY(cudaMalloc(&st->stage[slot], bytes));
    st->stage_bytes[slot] = bytes;
    return FA_OK;
}

}  // namespace
}  // namespace fa

using namespace fa;

namespace {
// fa_prefill with the kernel variant given (the host entry decides once for the whole problem so
// that its chunks of heads run the kernel a single launch would have run).
int prefill_on_device(const fa_prefill_args* a, int variant) {
    int rc = validate_prefill(a);
    if (rc != FA_OK) return rc;
    if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->o))
        return FA_ERR_MISALIGNED;
    if (a->lse && (reinterpret_cast<uintptr_t>(a->lse) & 3u)) return FA_ERR_MISALIGNED;
    DeviceState* st = device_state();
    if (!st) return FA_ERR_CUDA;
    if (st->cc_major != 10) return FA_ERR_NOT_SM100;
    if (a->dtype == FA_DTYPE_E4M3) return launch_prefill_fp8(*a, st);
    return launch_prefill_16bit(*a, st, variant);
}
}  // namespace

FA_EXPORT int fa_prefill(const fa_prefill_args* a) { return prefill_on_device(a, FA_PREFILL_AUTO); }

FA_EXPORT int fa_prefill_host(const fa_prefill_args* h) {
    int rc = validate_prefill(h);
    if (rc != FA_OK) return rc;
    DeviceState* st = device_state();
    if (!st) return FA_ERR_CUDA;
    // the staging buffers and the three streams belong to the device: one host call at a time
    std::lock_guard<std::mutex> host_lock(st->host_entry_mutex);
    const size_t bh    = (size_t)h->batch_size * h->num_heads;
    const size_t elems = bh * h->seq_len * h->d_head;
    const size_t in_b  = elems * (h->dtype == FA_DTYPE_E4M3 ? 1 : 2);
    const size_t out_b = elems * 2;
    const size_t lse_b = bh * h->seq_len * sizeof(float);
    const size_t sc_b  = bh * sizeof(float);
    // slots: 0 q, 1 k, 2 v, 3 o, 4 lse, 5..7 scales
    for (int s = 0; s < 3; s++)
        if ((rc = stage_reserve(st, s, in_b)) != FA_OK) return rc;
    if ((rc = stage_reserve(st, 3, out_b)) != FA_OK) return rc;
    if (h->lse && (rc = stage_reserve(st, 4, lse_b)) != FA_OK) return rc;
    for (int i = 0; i < 3; i++)
        if (!st->pipe[i]) FA_CUDA_TRY(cudaStreamCreateWithFlags(&st->pipe[i], cudaStreamNonBlocking));
    if (h->dtype == FA_DTYPE_E4M3) {
        const float* src[3] = {h->q_scale, h->k_scale, h->v_scale};
        for (int s = 0; s < 3; s++) {
            if ((rc = stage_reserve(st, 5 + s, sc_b)) != FA_OK) return rc;
            FA_CUDA_TRY(cudaMemcpy(st->stage[5 + s], src[s], sc_b, cudaMemcpyHostToDevice));
        }
    }
    // Heads are independent, so the batch*head axis is cut into chunks that flow through three
    // streams: while chunk i computes and its output goes back to the host, chunk i+1 is already
    // coming in.  Host-to-device (Q, K, V) and device-to-host (O, LSE) traffic use opposite PCIe
    // directions and overlap.  Chunks of >= ~2 MB per tensor keep the copies efficient (measured: 12 chunks beat 3 and 24).
    const size_t per_head_in = in_b / bh, per_head_out = out_b / bh, per_head_lse = lse_b / bh;
    size_t n_chunks = in_b / (2u << 20);
    if (n_chunks < 1) n_chunks = 1;
    if (n_chunks > 16) n_chunks = 16;
    if (n_chunks > bh) n_chunks = bh;
    const size_t heads_per_chunk = (bh + n_chunks - 1) / n_chunks;
    const int variant = choose_prefill_variant(h->batch_size, h->num_heads, h->seq_len, h->d_head, st);
    int ci = 0;
    for (size_t h0 = 0; h0 < bh; h0 += heads_per_chunk, ci++) {
        const size_t nh = (bh - h0 < heads_per_chunk) ? bh - h0 : heads_per_chunk;
        cudaStream_t stream = st->pipe[ci % 3];
        const char* hq = static_cast<const char*>(h->q) + h0 * per_head_in;
        const char* hk = static_cast<const char*>(h->k) + h0 * per_head_in;
        const char* hv = static_cast<const char*>(h->v) + h0 * per_head_in;
        char* dq = static_cast<char*>(st->stage[0]) + h0 * per_head_in;
        char* dk = static_cast<char*>(st->stage[1]) + h0 * per_head_in;
        char* dv = static_cast<char*>(st->stage[2]) + h0 * per_head_in;
        char* dO = static_cast<char*>(st->stage[3]) + h0 * per_head_out;
        FA_CUDA_TRY(cudaMemcpyAsync(dq, hq, nh * per_head_in, cudaMemcpyHostToDevice, stream));
        FA_CUDA_TRY(cudaMemcpyAsync(dk, hk, nh * per_head_in, cudaMemcpyHostToDevice, stream));
        FA_CUDA_TRY(cudaMemcpyAsync(dv, hv, nh * per_head_in, cudaMemcpyHostToDevice, stream));
        fa_prefill_args d = *h;
        d.q = dq; d.k = dk; d.v = dv; d.o = dO;
        d.lse = h->lse ? reinterpret_cast<float*>(static_cast<char*>(st->stage[4]) + h0 * per_head_lse) : nullptr;
        d.batch_size = 1;
        d.num_heads = static_cast<int>(nh);
        d.stream = stream;
        if (h->dtype == FA_DTYPE_E4M3) {
            d.q_scale = static_cast<float*>(st->stage[5]) + h0;
            d.k_scale = static_cast<float*>(st->stage[6]) + h0;
            d.v_scale = static_cast<float*>(st->stage[7]) + h0;
        }
        if ((rc = prefill_on_device(&d, variant)) != FA_OK) return rc;
        FA_CUDA_TRY(cudaMemcpyAsync(static_cast<char*>(h->o) + h0 * per_head_out, dO, nh * per_head_out,
                                    cudaMemcpyDeviceToHost, stream));
        if (h->lse)
            FA_CUDA_TRY(cudaMemcpyAsync(reinterpret_cast<char*>(h->lse) + h0 * per_head_lse,
                                        static_cast<char*>(st->stage[4]) + h0 * per_head_lse, nh * per_head_lse,
                                        cudaMemcpyDeviceToHost, stream));
    }
    for (int i = 0; i < 3; i++) FA_CUDA_TRY(cudaStreamSynchronize(st->pipe[i]));
    int word = 0;
    FA_CUDA_TRY(cudaMemcpy(&word, st->status, sizeof(int), cudaMemcpyDeviceToHost));
    return status_word_to_error(word);
}

FA_EXPORT int fa_device_status(int* status_word) {
    DeviceState* st = device_state();
    if (!st) return FA_ERR_CUDA;
    FA_CUDA_TRY(cudaDeviceSynchronize());
    int word = 0;
    FA_CUDA_TRY(cudaMemcpy(&word, st->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (status_word) *status_word = word;
    return status_word_to_error(word);
}

FA_EXPORT int fa_status_word_to_error(int status_word) { return status_word_to_error(status_word); }

FA_EXPORT int fa_clear_device_status(void) {
    DeviceState* st = device_state();
    if (!st) return FA_ERR_CUDA;
    FA_CUDA_TRY(cudaDeviceSynchronize());
    FA_CUDA_TRY(cudaMemset(st->status, 0, sizeof(int)));
    return FA_OK;
}

FA_EXPORT const char* fa_error_string(int code) {
    switch (code) {
        case FA_OK:                   return "ok";
        case FA_ERR_INVALID_ARGUMENT: return "invalid argument";
        case FA_ERR_UNSUPPORTED:      return "unsupported d_head, dtype or split count";
        case FA_ERR_MISALIGNED:       return "device pointer not 16-byte aligned";
        case FA_ERR_WORKSPACE:        return "workspace missing or too small";
        case FA_ERR_CUDA:             return "CUDA call failed";
        case FA_ERR_DEVICE_TIMEOUT:   return "a kernel gave up on a bounded wait";
        case FA_ERR_NOT_SM100:        return "device is not compute capability 10.x";
        case FA_ERR_NCCL:             return "NCCL call failed or libnccl not found";
        default:                      return "unknown error";
    }
}

FA_EXPORT int fa_set_prefill_variant(int variant) {
    if (variant != FA_PREFILL_AUTO && variant != FA_PREFILL_ONE_TILE && variant != FA_PREFILL_TILE_PAIR &&
        variant != FA_PREFILL_CTA_PAIR)
        return FA_ERR_INVALID_ARGUMENT;
    g_prefill_variant.store(variant, std::memory_order_relaxed);
    return FA_OK;
}

FA_EXPORT const char* fa_last_cuda_error(void) { return g_last_cuda_error; }
FA_EXPORT int fa_version(void) { return 100; }

// ---------------------------------------------------------------------------
// The reference's C++ entry point.  Same contract as
// kernels/flash_attention.cu:595-617: enqueue on params.stream, return without
// synchronising; any failure prints to stderr and exits, as CUDA_CHECK does in
// the reference (include/flash_attention.h:35-43).
// ---------------------------------------------------------------------------
namespace transformer {

__attribute__((visibility("default")))
void launch_flash_attention(const FlashAttentionParams& params) {
    fa_prefill_args a;
    std::memset(&a, 0, sizeof(a));
    a.q = params.Q; a.k = params.K; a.v = params.V; a.o = params.O; a.lse = params.L;
    a.batch_size = params.batch_size;
    a.num_heads  = params.num_heads;
    a.seq_len    = params.seq_len;
    a.d_head     = params.d_head;
    a.scale      = params.scale;
    a.causal     = params.causal ? 1 : 0;
    a.dtype      = params.dtype == 1 ? FA_DTYPE_BF16 : FA_DTYPE_F16;
    a.stream     = params.stream;
    const int rc = fa_prefill(&a);
    if (rc != FA_OK) {
        fprintf(stderr, "launch_flash_attention: %s%s%s\n", fa_error_string(rc),
                rc == FA_ERR_CUDA ? ": " : "", rc == FA_ERR_CUDA ? fa_last_cuda_error() : "");
        exit(EXIT_FAILURE);
    }
}

}  // namespace transformer
