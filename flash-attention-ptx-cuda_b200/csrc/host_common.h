// Host-side plumbing shared by the entry points: per-device state (SM count,
// status word, staging buffers), the tensor-map encoder and error bookkeeping.
//
// The reference caches one SM count for the whole process
// (kernels/flash_attention.cu:582-591, get_sm_count); here the state is kept
// per device so that one process can drive several GPUs.
#pragma once

#include <atomic>
#include <cstddef>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/fa_b200.h"

#define FA_EXPORT extern "C" __attribute__((visibility("default")))

namespace fa {

struct DeviceState {
    std::atomic<bool> ready{false};  // set last, with release order, by the thread that filled the fields in
    std::mutex host_entry_mutex;     // serialises fa_prefill_host calls on this device (shared staging and streams)
    int    device      = -1;
    int    sm_count    = 0;
    int    cc_major    = 0;
    int*   status      = nullptr;   // device int, error word written by kernels
    void*  stage[8]    = {};        // host-entry staging buffers (device memory)
    size_t stage_bytes[8] = {};
    cudaStream_t pipe[3] = {};      // host-entry streams: chunks of heads are copied in, computed
                                    // and copied out on alternating streams so the two PCIe
                                    // directions and the kernels overlap
    // e4m3 prefill: memory pool of the library's own for the stream-ordered fp16 copy of V (created
    // at the first such call; keeps what it has allocated, so later calls allocate nothing new)
    std::atomic<bool> pool_ready{false};
    std::mutex pool_mutex;
    cudaMemPool_t scratch_pool = nullptr;
};

// State of the current device (created on first use).  nullptr on CUDA failure.
DeviceState* device_state();

// Remembers a CUDA failure for fa_last_cuda_error() and returns FA_ERR_CUDA.
int note_cuda_error(cudaError_t err, const char* where);
int note_driver_error(CUresult err, const char* where);
// Remembers `msg` for fa_last_cuda_error() and returns `code`.
int note_message(const char* msg, int code);

#define FA_CUDA_TRY(expr)                                               \
    do {                                                                \
        cudaError_t fa_try_err_ = (expr);                               \
        if (fa_try_err_ != cudaSuccess) return ::fa::note_cuda_error(fa_try_err_, #expr); \
    } while (0)

// Rank-3 tiled tensor map over a dense [n_heads, n_rows, row_elems] tensor with
// 128-byte swizzle.  box_cols * elem_bytes must be 128; box_rows <= 256.
// dtype is an FA_DTYPE_* value.
int make_tensor_map_3d(CUtensorMap* out, const void* base, int dtype, uint64_t row_elems,
                       uint64_t n_rows, uint64_t n_heads, uint32_t box_cols, uint32_t box_rows);

// Rank-4 tiled tensor map over a KV cache: dims (row_elems, n_rows, n_heads, n_blocks) with the
// three outer strides given in ELEMENTS (each a multiple of 8); 128-byte swizzle, box
// (box_cols, box_rows, 1, 1).  Rows past n_rows read as zero.
int make_tensor_map_4d(CUtensorMap* out, const void* base, int dtype, uint64_t row_elems,
                       uint64_t n_rows, uint64_t n_heads, uint64_t n_blocks, uint64_t row_stride,
                       uint64_t head_stride, uint64_t block_stride, uint32_t box_cols, uint32_t box_rows);

// Rank-5 tensor map over the decode queries [B, T, Hq, D] seen as (d, head in group, token, KV head,
// batch): one box holds the `group` x `n_tok` rows of a (batch, KV head) pair, token-major.
int make_tensor_map_q5(CUtensorMap* out, const void* base, int dtype, uint64_t d_head, uint64_t group,
                       uint64_t n_tok, uint64_t n_kv_heads, uint64_t batch, uint32_t box_cols);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Implemented next to their kernels.
// `variant` is an FA_PREFILL_* value; FA_PREFILL_AUTO decides from the sizes in `a`.
int launch_prefill_16bit(const fa_prefill_args& a, DeviceState* st, int variant);
int choose_prefill_variant(int batch_size, int num_heads, int seq_len, int d_head, const DeviceState* st);
// The kernel on pairs of CTAs (d_head 128): builds its own tensor maps (half-tile boxes for K).
int launch_prefill_2sm_16bit(const fa_prefill_args& a, DeviceState* st, int heads_per_group);
int launch_prefill_fp8(const fa_prefill_args& a, DeviceState* st);
// The kernel with two query tiles per CTA (tensor maps as for the one-tile kernel).
int launch_prefill_pair_16bit(const fa_prefill_args& a, DeviceState* st, int heads_per_group, const CUtensorMap& tq,
                              const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to);
// FA_PREFILL_* choice made through fa_set_prefill_variant().
extern std::atomic<int> g_prefill_variant;

// Grouped-query decode on the prefill kernel: the `group` query heads that share a KV head ride
// in the rows of one query tile; work items are (batch x KV head, KV split).
struct GqaLaunch {
    const void* q; const void* k; const void* v;
    float* o_part; float* lse_part;           // [row][split][D] and [row][split], row = (b * T + t) * Hq + hq
    void* o_final; float* lse_final;          // the caller's o / lse: written directly when n_splits == 1
    int batch, n_kv_heads, group, kv_len, d_head, dtype;
    int n_tok;                                // query tokens per sequence (1 = plain decode)
    int n_splits, tiles_per_split;
    long long row_stride, head_stride, batch_stride;   // of the KV cache, in elements
    const int* seq_lens;                      // [batch] or null
    const int* block_table;                   // paged cache: [batch][table_stride] page numbers, or null
    int table_stride, page_size, n_pages;
    long long page_stride;                    // elements between pages
    const float* q_scale; const float* k_scale; const float* v_scale;   // e4m3: per (batch, KV head)
    float scale;
    cudaStream_t stream;
};
int launch_decode_gqa(const GqaLaunch& g, DeviceState* st);

}  // namespace fa
