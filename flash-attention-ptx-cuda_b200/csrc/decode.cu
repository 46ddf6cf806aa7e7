// Split-KV decode (one query row per head against a long KV cache) and the LSE
// merge ("combine") kernel.
//
// The reference has no decode path; the definition is its attention
// (src/demo.cu:28-70) evaluated for a single query row, every key visible.  At
// one query row the work is one multiply-add per byte of K and V read, so the
// kernels here are built around HBM traffic, not tensor cores:
//
//   decode_partial_kernel  grid batch*heads x splits (one-dimensional).  Each warp streams rows
//     of K and V straight from global memory with 128-bit loads (a 16-lane group
//     covers one 256-byte row at d_head 128, so every warp instruction reads
//     whole rows, fully coalesced), keeps an online softmax (running max, sum,
//     fp32 accumulator slice) per lane group in registers, and never touches
//     shared memory until the per-CTA merge at the end.  Output per (head,
//     split): a normalised fp32 partial O and its natural-log LSE.
//   combine_kernel  merges partials by their LSEs,
//       m = max lse_p, w_p = exp(lse_p - m), O = sum w_p O_p / sum w_p,
//       LSE = m + log(sum w_p),
//     converts to the 16-bit output type, and can also emit the fp32 result.
//     The same kernel merges the per-GPU partials of KV-sequence-sharded decode
//     (parts = ranks), reading the gathered buffer directly.
#include <cfloat>
#include <cmath>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <dlfcn.h>
#include <nccl.h>

#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "host_common.h"

namespace fa {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2   = 0.6931471805599453f;
constexpr int   kDecodeWarps = 8;
constexpr int   kUnroll = 4;            // row groups in flight per warp iteration

__device__ __forceinline__ uint4 ld_stream_16(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
    if constexpr (BF16) {
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
    } else {
        return __half22float2(*reinterpret_cast<const __half2*>(&w));
    }
}

template <bool BF16>
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    float2 a = unpack2<BF16>(u.x), b = unpack2<BF16>(u.y), c = unpack2<BF16>(u.z), d = unpack2<BF16>(u.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

__device__ __forceinline__ float fast_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Merges two online-softmax states (m in log2 units).
__device__ __forceinline__ void merge_state(float& m, float& l, float (&acc)[8], float m2, float l2,
                                            const float (&acc2)[8]) {
    const float mn = fmaxf(m, m2);
    const float c1 = fast_ex2(m - mn), c2 = fast_ex2(m2 - mn);
    l = l * c1 + l2 * c2;
#pragma unroll
    for (int e = 0; e < 8; e++) acc[e] = acc[e] * c1 + acc2[e] * c2;
    m = mn;
}

template <int D, bool BF16>
__global__ void __launch_bounds__(kDecodeWarps * 32)
decode_partial_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ k,
                      const uint16_t* __restrict__ v, float* __restrict__ o_part,
                      float* __restrict__ lse_part, int seq_len_kv, int n_splits, int keys_per_split,
                      float scale_log2) {
    constexpr int LPR = D / 8;           // lanes covering one row (8 elements = 16 bytes per lane)
    constexpr int RPW = 32 / LPR;        // rows per warp-wide load
    constexpr int STEP = kDecodeWarps * RPW;
    // one-dimensional grid: the splits of a head are neighbours, and batch * heads is not limited to 65535
    const int bh = blockIdx.x / n_splits, split = blockIdx.x - bh * n_splits;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / LPR;          // which row of the warp-wide load this lane reads
    const int dsl = (lane % LPR) * 8;    // first of this lane's 8 head-dim elements
    const int k_begin = split * keys_per_split;
    const int k_end = min(seq_len_kv, k_begin + keys_per_split);

    float qf[8];
    {
        const uint4 qu = *reinterpret_cast<const uint4*>(q + (size_t)bh * D + dsl);
        unpack8<BF16>(qu, qf);
#pragma unroll
        for (int e = 0; e < 8; e++) qf[e] *= scale_log2;
    }
    const uint16_t* kb = k + ((size_t)bh * seq_len_kv) * D + dsl;
    const uint16_t* vb = v + ((size_t)bh * seq_len_kv) * D + dsl;

    float m = -1e30f, l = 0.0f, acc[8];
#pragma unroll
    for (int e = 0; e < 8; e++) acc[e] = 0.0f;

    for (int base = k_begin; base < k_end; base += kUnroll * STEP) {
        // This lane's rows of the iteration: r0, r0 + STEP, ... (kUnroll of them).
        const int r0 = base + warp * RPW + sub;
        uint4 ku[kUnroll], vu[kUnroll];
        bool valid[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            const int r = r0 + u * STEP;
            valid[u] = r < k_end;
            const size_t off = (size_t)(valid[u] ? r : k_begin) * D;
            ku[u] = ld_stream_16(kb + off);
            vu[u] = ld_stream_16(vb + off);
        }
        float s[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            float kf[8];
            unpack8<BF16>(ku[u], kf);
            float d = 0.0f;
#pragma unroll
            for (int e = 0; e < 8; e++) d = fmaf(qf[e], kf[e], d);
#pragma unroll
            for (int o = 1; o < LPR; o <<= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
            s[u] = valid[u] ? d : -INFINITY;
        }
        float mn = m;
#pragma unroll
        for (int u = 0; u < kUnroll; u++) mn = fmaxf(mn, s[u]);
        const float corr = fast_ex2(m - mn);
        m = mn;
        l *= corr;
#pragma unroll
        for (int e = 0; e < 8; e++) acc[e] *= corr;
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            const float p = fast_ex2(s[u] - mn);
            l += p;
            float vf[8];
            unpack8<BF16>(vu[u], vf);
#pragma unroll
            for (int e = 0; e < 8; e++) acc[e] = fmaf(p, vf[e], acc[e]);
        }
    }

    // Merge the RPW lane groups of the warp (they hold the same d-slice of different rows).
#pragma unroll
    for (int o = LPR; o < 32; o <<= 1) {
        float m2 = __shfl_xor_sync(0xffffffffu, m, o);
        float l2 = __shfl_xor_sync(0xffffffffu, l, o);
        float a2[8];
#pragma unroll
        for (int e = 0; e < 8; e++) a2[e] = __shfl_xor_sync(0xffffffffu, acc[e], o);
        merge_state(m, l, acc, m2, l2, a2);
    }
    // Merge the warps of the CTA through shared memory.
    __shared__ float sm_m[kDecodeWarps], sm_l[kDecodeWarps];
    __shared__ float sm_acc[kDecodeWarps][D];
    if (lane < LPR) {
#pragma unroll
        for (int e = 0; e < 8; e++) sm_acc[warp][dsl + e] = acc[e];
        if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
    }
    __syncthreads();
    if (threadIdx.x < D) {
        const int d = threadIdx.x;
        float mm = -1e30f;
#pragma unroll
        for (int w = 0; w < kDecodeWarps; w++) mm = fmaxf(mm, sm_m[w]);
        float ll = 0.0f, a = 0.0f;
#pragma unroll
        for (int w = 0; w < kDecodeWarps; w++) {
            const float c = fast_ex2(sm_m[w] - mm);
            ll += sm_l[w] * c;
            a += sm_acc[w][d] * c;
        }
        const size_t pidx = (size_t)bh * n_splits + split;
        o_part[pidx * D + d] = ll > 0.0f ? a / ll : 0.0f;
        if (d == 0) lse_part[pidx] = ll > 0.0f ? kLn2 * (mm + log2f(ll)) : -INFINITY;
    }
}

// One CTA per output row, one thread per head-dim element.  Inputs and the fp32 output are
// addressed by strides, so the same kernel reads split partials ([row][split][D]), gathered
// per-rank partials ([rank][row][D]) and packed ones ([rank][row][D + 1], LSE in the last
// column), and can write a packed row itself.
template <bool BF16>
__global__ void combine_kernel(const float* __restrict__ o_parts, const float* __restrict__ lse_parts,
                               int n_parts, long long part_stride_o, long long row_stride_o,
                               long long part_stride_l, long long row_stride_l, int d_head,
                               uint16_t* __restrict__ o, float* __restrict__ lse, long long lse_stride,
                               float* __restrict__ o_f32, long long o_f32_stride) {
    const int row = blockIdx.x, d = threadIdx.x;
    const float* lp = lse_parts + (size_t)row * row_stride_l;
    float m = -INFINITY;
    for (int p = 0; p < n_parts; p++) m = fmaxf(m, lp[(size_t)p * part_stride_l]);
    float wsum = 0.0f, a = 0.0f;
    if (m > -INFINITY) {
        const float* op = o_parts + (size_t)row * row_stride_o + d;
        for (int p = 0; p < n_parts; p++) {
            const float w = fast_ex2((lp[(size_t)p * part_stride_l] - m) * kLog2e);
            wsum += w;
            a = fmaf(w, op[(size_t)p * part_stride_o], a);
        }
    }
    const float out = wsum > 0.0f ? a / wsum : 0.0f;
    if (o != nullptr) {
        uint16_t bits;
        if constexpr (BF16) bits = __bfloat16_as_ushort(__float2bfloat16_rn(out));
        else bits = __half_as_ushort(__float2half_rn(out));
        o[(size_t)row * d_head + d] = bits;
    }
    if (o_f32 != nullptr) o_f32[(size_t)row * o_f32_stride + d] = out;
    if (lse != nullptr && d == 0) lse[(size_t)row * lse_stride] = wsum > 0.0f ? m + kLn2 * log2f(wsum) : -INFINITY;
}

// A rank that holds no key of a KV-sequence-sharded cache contributes weight zero to the merge.
__global__ void empty_partial_kernel(float* packed, int d_head) {
    float* row = packed + (size_t)blockIdx.x * (d_head + 1);
    row[threadIdx.x] = 0.0f;
    if (threadIdx.x == 0) row[d_head] = -INFINITY;
}

struct CombineOut {
    void*     o = nullptr;           // 16-bit [rows][D], optional
    float*    lse = nullptr;         // optional
    long long lse_stride = 1;
    float*    o_f32 = nullptr;       // optional
    long long o_f32_stride = 0;
};

int launch_combine(const float* o_parts, const float* lse_parts, int n_parts, long long pso,
                   long long rso, long long psl, long long rsl, int rows, int d_head, const CombineOut& out,
                   int dtype, cudaStream_t stream) {
    if (dtype == FA_DTYPE_BF16)
        combine_kernel<true><<<rows, d_head, 0, stream>>>(o_parts, lse_parts, n_parts, pso, rso, psl, rsl, d_head,
                                                          static_cast<uint16_t*>(out.o), out.lse, out.lse_stride,
                                                          out.o_f32, out.o_f32_stride);
    else
        combine_kernel<false><<<rows, d_head, 0, stream>>>(o_parts, lse_parts, n_parts, pso, rso, psl, rsl, d_head,
                                                           static_cast<uint16_t*>(out.o), out.lse, out.lse_stride,
                                                           out.o_f32, out.o_f32_stride);
    FA_CUDA_TRY(cudaGetLastError());
    return FA_OK;
}

size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

int default_splits(int sms, long long bh, int seq_len_kv) {
    // Enough CTAs for ~8 per SM, but never fewer than 512 keys per split.
    long long want = (8ll * sms + bh - 1) / bh;
    long long max_by_len = seq_len_kv / 512 > 0 ? seq_len_kv / 512 : 1;
    long long s = want < max_by_len ? want : max_by_len;
    if (s < 1) s = 1;
    if (s > FA_MAX_SPLITS) s = FA_MAX_SPLITS;
    return (int)s;
}

// Argument checks shared by every entry point that takes fa_decode_args.
int validate_decode(const fa_decode_args* a, bool need_output) {
    if (!a || !a->q || !a->k || !a->v) return FA_ERR_INVALID_ARGUMENT;
    if (need_output) {
        if (!a->o && !a->o_f32) return FA_ERR_INVALID_ARGUMENT;
        if (a->o_f32 && !a->lse) return FA_ERR_INVALID_ARGUMENT;
    }
    if (a->batch_size <= 0 || a->num_heads <= 0 || a->seq_len_kv <= 0) return FA_ERR_INVALID_ARGUMENT;
    if (!(a->scale > 0.0f) || !std::isfinite(a->scale)) return FA_ERR_INVALID_ARGUMENT;
    if (a->dtype != FA_DTYPE_F16 && a->dtype != FA_DTYPE_BF16) return FA_ERR_UNSUPPORTED;
    if (a->d_head != 64 && a->d_head != 128) return FA_ERR_UNSUPPORTED;
    if (a->num_splits < 0 || a->num_splits > FA_MAX_SPLITS) return FA_ERR_UNSUPPORTED;
    const long long bh = (long long)a->batch_size * a->num_heads;
    if (bh * FA_MAX_SPLITS > 0x7FFFFFFFll) return FA_ERR_UNSUPPORTED;   // grid.x
    if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || (a->o && !aligned16(a->o)))
        return FA_ERR_MISALIGNED;
    return FA_OK;
}

// The split count actually used: the caller's or the default, with no empty trailing split.
void plan_splits(const fa_decode_args* a, int sm_count, int* splits_out, int* keys_per_split_out) {
    const long long bh = (long long)a->batch_size * a->num_heads;
    int splits = a->num_splits ? a->num_splits : default_splits(sm_count, bh, a->seq_len_kv);
    if (splits > a->seq_len_kv) splits = a->seq_len_kv;
    const int kps = (a->seq_len_kv + splits - 1) / splits;
    *splits_out = (a->seq_len_kv + kps - 1) / kps;
    *keys_per_split_out = kps;
}

// The two launches of a decode step: per-split partials into `scratch` (fp32 O [bh][split][D], then,
// 256-byte aligned, LSE [bh][split]), and their merge into `out`.  Shared by fa_decode (caller's
// workspace), fa_decode_static (the built-in array) and the KV-sharded entry (packed output).
int decode_into(const fa_decode_args* a, int splits, int kps, void* scratch, const CombineOut& out) {
    const long long bh = (long long)a->batch_size * a->num_heads;
    float* o_part = static_cast<float*>(scratch);
    float* lse_part = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) +
                                               align256((size_t)bh * splits * a->d_head * sizeof(float)));
    cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
    const unsigned grid = (unsigned)(bh * splits);
    const float sl2 = a->scale * kLog2e;
    const uint16_t* q = static_cast<const uint16_t*>(a->q);
    const uint16_t* k = static_cast<const uint16_t*>(a->k);
    const uint16_t* v = static_cast<const uint16_t*>(a->v);
    const bool bf = a->dtype == FA_DTYPE_BF16;
#define FA_LAUNCH_DECODE(DH, BF) \
    decode_partial_kernel<DH, BF><<<grid, kDecodeWarps * 32, 0, stream>>>(q, k, v, o_part, lse_part, \
        a->seq_len_kv, splits, kps, sl2)
    if (a->d_head == 128) { if (bf) FA_LAUNCH_DECODE(128, true); else FA_LAUNCH_DECODE(128, false); }
    else                  { if (bf) FA_LAUNCH_DECODE(64, true);  else FA_LAUNCH_DECODE(64, false); }
#undef FA_LAUNCH_DECODE
    FA_CUDA_TRY(cudaGetLastError());
    // partials: o [bh][split][D], lse [bh][split]
    return launch_combine(o_part, lse_part, splits, a->d_head, (long long)splits * a->d_head, 1, splits,
                          (int)bh, a->d_head, out, a->dtype, stream);
}

CombineOut caller_outputs(const fa_decode_args* a) {
    CombineOut out;
    out.o = a->o; out.lse = a->lse; out.lse_stride = 1;
    out.o_f32 = a->o_f32; out.o_f32_stride = a->d_head;
    return out;
}

}  // namespace
}  // namespace fa

using namespace fa;

FA_EXPORT size_t fa_decode_workspace_bytes(int batch_size, int num_heads, int d_head, int num_splits) {
    if (batch_size <= 0 || num_heads <= 0 || d_head <= 0 || num_splits <= 0) return 0;
    const size_t parts = (size_t)batch_size * num_heads * num_splits;
    return align256(parts * d_head * sizeof(float)) + align256(parts * sizeof(float));
}

FA_EXPORT int fa_decode_default_splits(int batch_size, int num_heads, int seq_len_kv) {
    if (batch_size <= 0 || num_heads <= 0 || seq_len_kv <= 0) return 0;
    DeviceState* st = device_state();
    return default_splits(st ? st->sm_count : 148, (long long)batch_size * num_heads, seq_len_kv);
}

FA_EXPORT int fa_decode(const fa_decode_args* a) {
    int rc = validate_decode(a, true);
    if (rc != FA_OK) return rc;
    DeviceState* st = device_state();
    if (!st) return FA_ERR_CUDA;
    if (st->cc_major != 10) return FA_ERR_NOT_SM100;
    int splits, kps;
    plan_splits(a, st->sm_count, &splits, &kps);
    const size_t need = fa_decode_workspace_bytes(a->batch_size, a->num_heads, a->d_head, splits);
    if (!a->workspace || a->workspace_bytes < need || !aligned16(a->workspace)) return FA_ERR_WORKSPACE;
    return decode_into(a, splits, kps, a->workspace, caller_outputs(a));
}

// ---------------------------------------------------------------------------
// fa_decode_static: split-KV decode for callers that may not allocate.
//
// The partial (O, LSE) results go to the file-scope device array below instead
// of a caller-provided workspace.  In host code the array's name is only a
// handle, not a device address, so the address is looked up once per device
// with cudaGetSymbolAddress (with that device current) and that pointer is what
// the kernels receive.  Nothing on this path allocates: it does not touch the
// per-device state used by the other entry points (that state owns a
// cudaMalloc'ed status word), it queries the device attributes directly.
// ---------------------------------------------------------------------------
namespace fa {
namespace {

static __device__ __align__(256) unsigned char g_decode_static_scratch[FA_DECODE_STATIC_SCRATCH_BYTES];

struct StaticScratchSetup {
    std::atomic<bool> ready{false};   // release-stored after the fields below, acquire-loaded before them
    void* ptr = nullptr;              // device address of g_decode_static_scratch on this device
    int   cc_major = 0;
    int   sm_count = 0;
};
StaticScratchSetup g_static_setup[64];
std::mutex g_static_mutex;

// First call on a device: check the device, then resolve the array's device address.
int static_scratch_setup(StaticScratchSetup** out) {
    int dev = 0;
    FA_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return FA_ERR_INVALID_ARGUMENT;
    StaticScratchSetup* s = &g_static_setup[dev];
    if (!s->ready.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (!s->ready.load(std::memory_order_relaxed)) {
            int major = 0, sms = 0;
            FA_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
            FA_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
            // before the symbol lookup: on another architecture the library holds no image for the
            // device and the lookup would fail with a less helpful error
            if (major != 10) return FA_ERR_NOT_SM100;
            void* ptr = nullptr;
            FA_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_decode_static_scratch));
            s->ptr = ptr;
            s->cc_major = major;
            s->sm_count = sms;
            s->ready.store(true, std::memory_order_release);
        }
    }
    *out = s;
    return FA_OK;
}

}  // namespace
}  // namespace fa

FA_EXPORT int fa_decode_static(const fa_decode_args* a) {
    int rc = validate_decode(a, true);
    if (rc != FA_OK) return rc;
    StaticScratchSetup* su = nullptr;
    rc = static_scratch_setup(&su);
    if (rc != FA_OK) return rc;
    int splits, kps;
    plan_splits(a, su->sm_count, &splits, &kps);
    if (fa_decode_workspace_bytes(a->batch_size, a->num_heads, a->d_head, splits) >
        (size_t)FA_DECODE_STATIC_SCRATCH_BYTES)
        return FA_ERR_WORKSPACE;
    return decode_into(a, splits, kps, su->ptr, caller_outputs(a));
}

// ---------------------------------------------------------------------------
// fa_decode_gqa: grouped-query decode.  The partial pass is the prefill kernel in
// its grouped-query mode (tcgen05: the query heads of a group are the rows of
// the query tile); the merge over KV splits is combine_kernel.
// ---------------------------------------------------------------------------
namespace {
// Number of KV splits: the persistent kernel runs ceil(items / SMs) rounds of equal items, an
// item costs its key tiles plus about two tiles of hand-over, so take the split count with the
// smallest rounds x (tiles per split + 2); at least 4 key tiles (512 keys) per split.  The
// same value for every caller of the same shape.
int gqa_splits(int sms, long long bh_kv, int seq_len_kv) {
    const int n_tiles = (seq_len_kv + 127) / 128;
    int cap = n_tiles / 4 > 0 ? n_tiles / 4 : 1;
    if (cap > FA_MAX_SPLITS) cap = FA_MAX_SPLITS;
    long long best_cost = -1;
    int best = 1;
    for (int s = 1; s <= cap; s++) {
        const int tps = (n_tiles + s - 1) / s;
        const int s_eff = (n_tiles + tps - 1) / tps;     // no empty trailing split
        const long long rounds = (bh_kv * s_eff + sms - 1) / sms;
        const long long cost = rounds * (tps + 2);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = s_eff; }
    }
    return best;
}
}  // namespace

FA_EXPORT int fa_decode_gqa_default_splits(int batch_size, int num_kv_heads, int seq_len_kv) {
    if (batch_size <= 0 || num_kv_heads <= 0 || seq_len_kv <= 0) return 0;
    DeviceState* st = device_state();
    return gqa_splits(st ? st->sm_count : 148, (long long)batch_size * num_kv_heads, seq_len_kv);
}

FA_EXPORT int fa_decode_gqa(const fa_decode_gqa_args* a) {
    if (!a || !a->q || !a->k || !a->v || !a->o) return FA_ERR_INVALID_ARGUMENT;
    if (a->batch_size <= 0 || a->num_q_heads <= 0 || a->num_kv_heads <= 0 || a->seq_len_kv <= 0)
        return FA_ERR_INVALID_ARGUMENT;
    if (a->num_q_heads % a->num_kv_heads != 0) return FA_ERR_INVALID_ARGUMENT;
    if (!(a->scale > 0.0f) || !std::isfinite(a->scale)) return FA_ERR_INVALID_ARGUMENT;
    if (a->dtype != FA_DTYPE_F16 && a->dtype != FA_DTYPE_BF16 && a->dtype != FA_DTYPE_E4M3) return FA_ERR_UNSUPPORTED;
    if (a->d_head != 64 && a->d_head != 128) return FA_ERR_UNSUPPORTED;
    const bool e4m3 = a->dtype == FA_DTYPE_E4M3;
    if (e4m3) {                                         // e4m3 cache and query, per-(batch, KV head) scales, bf16 out
        if (a->d_head != 128) return FA_ERR_UNSUPPORTED;
        if (!a->q_scale || !a->k_scale || !a->v_scale) return FA_ERR_INVALID_ARGUMENT;
    }
    const int align_elems = e4m3 ? 16 : 8;              // strides are multiples of 16 bytes
    if (a->num_splits < 0 || a->num_splits > FA_MAX_SPLITS) return FA_ERR_UNSUPPORTED;
    const int group = a->num_q_heads / a->num_kv_heads;
    const int n_tok = a->num_q_tokens > 0 ? a->num_q_tokens : 1;
    if (a->num_q_tokens < 0 || n_tok > a->seq_len_kv) return FA_ERR_INVALID_ARGUMENT;
    if (group > 128) return FA_ERR_UNSUPPORTED;                         // the group must fit one query tile

    const long long rows = (long long)a->batch_size * n_tok * a->num_q_heads;
    if (rows > 0x7FFFFFFFll) return FA_ERR_INVALID_ARGUMENT;
    long long rs = a->kv_row_stride, hs = a->kv_head_stride, bs = a->kv_batch_stride;
    if (rs == 0 && hs == 0 && bs == 0) {               // dense [B, Hkv, Skv, D]
        rs = a->d_head;
        hs = (long long)a->seq_len_kv * a->d_head;
        bs = hs * a->num_kv_heads;
    }
    const bool paged = a->block_table != nullptr;
    if (paged) {
        const int ps = a->page_size;
        if (ps < 16 || (ps & (ps - 1)) != 0 || a->num_pages <= 0) return FA_ERR_INVALID_ARGUMENT;
        if ((long long)a->block_table_stride * ps < a->seq_len_kv) return FA_ERR_INVALID_ARGUMENT;
        if (a->kv_row_stride < a->d_head || a->kv_head_stride <= 0 || a->kv_page_stride <= 0)
            return FA_ERR_INVALID_ARGUMENT;
        if ((a->kv_row_stride % align_elems) || (a->kv_head_stride % align_elems) || (a->kv_page_stride % align_elems))
            return FA_ERR_MISALIGNED;
        rs = a->kv_row_stride; hs = a->kv_head_stride; bs = 16;
    }
    if (rs < a->d_head || hs <= 0 || bs <= 0) return FA_ERR_INVALID_ARGUMENT;
    if ((rs % align_elems) || (hs % align_elems) || (bs % align_elems)) return FA_ERR_MISALIGNED;
    if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->o)) return FA_ERR_MISALIGNED;
    DeviceState* st = device_state();
    if (!st) return FA_ERR_CUDA;
    if (st->cc_major != 10) return FA_ERR_NOT_SM100;

    const int n_tiles = (a->seq_len_kv + 127) / 128;
    const int tok_per_tile = 128 / group < n_tok ? 128 / group : n_tok;
    const int n_qt = (n_tok + tok_per_tile - 1) / tok_per_tile;     // query tiles per (batch, KV head)
    int splits = a->num_splits ? a->num_splits
                               : gqa_splits(st->sm_count, (long long)a->batch_size * a->num_kv_heads * n_qt, a->seq_len_kv);
    if (splits > n_tiles) splits = n_tiles;
    const int tps = (n_tiles + splits - 1) / splits;
    splits = (n_tiles + tps - 1) / tps;
    const size_t need = fa_decode_workspace_bytes(a->batch_size, n_tok * a->num_q_heads, a->d_head, splits);
    if (!a->workspace || a->workspace_bytes < need || !aligned16(a->workspace)) return FA_ERR_WORKSPACE;
    float* o_part = static_cast<float*>(a->workspace);
    float* lse_part = reinterpret_cast<float*>(static_cast<uint8_t*>(a->workspace) +
                                               align256((size_t)rows * splits * a->d_head * sizeof(float)));
    cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
    GqaLaunch g{};
    g.n_tok = n_tok;
    g.q = a->q; g.k = a->k; g.v = a->v;
    g.o_part = o_part; g.lse_part = lse_part;
    g.o_final = a->o; g.lse_final = a->lse;
    g.batch = a->batch_size; g.n_kv_heads = a->num_kv_heads; g.group = group;
    g.kv_len = a->seq_len_kv; g.d_head = a->d_head; g.dtype = a->dtype;
    g.n_splits = splits; g.tiles_per_split = tps;
    g.row_stride = rs; g.head_stride = hs; g.batch_stride = bs;
    g.seq_lens = a->seq_lens;
    g.block_table = a->block_table; g.table_stride = a->block_table_stride;
    g.page_size = paged ? a->page_size : 0; g.n_pages = a->num_pages; g.page_stride = a->kv_page_stride;
    g.q_scale = a->q_scale; g.k_scale = a->k_scale; g.v_scale = a->v_scale;
    g.scale = a->scale; g.stream = stream;
    int rc = launch_decode_gqa(g, st);
    if (rc != FA_OK) return rc;
    if (splits == 1) return FA_OK;                      // the kernel wrote o and lse itself
    CombineOut out;
    out.o = a->o; out.lse = a->lse;
    return launch_combine(o_part, lse_part, splits, a->d_head, (long long)splits * a->d_head, 1, splits,
                          (int)rows, a->d_head, out, e4m3 ? FA_DTYPE_BF16 : a->dtype, stream);
}

FA_EXPORT int fa_combine(const float* o_parts, const float* lse_parts, int n_parts, int rows,
                         int d_head, void* o, float* lse, int dtype, void* stream) {
    if (!o_parts || !lse_parts || !o || n_parts <= 0 || rows <= 0) return FA_ERR_INVALID_ARGUMENT;
    if (d_head != 64 && d_head != 128) return FA_ERR_UNSUPPORTED;
    if (dtype != FA_DTYPE_F16 && dtype != FA_DTYPE_BF16) return FA_ERR_UNSUPPORTED;
    DeviceState* st = device_state();
    if (!st) return FA_ERR_CUDA;
    // gathered layout: o [part][row][D], lse [part][row]
    CombineOut out;
    out.o = o; out.lse = lse;
    return launch_combine(o_parts, lse_parts, n_parts, (long long)rows * d_head, d_head, rows, 1, rows,
                          d_head, out, dtype, static_cast<cudaStream_t>(stream));
}

FA_EXPORT int fa_combine_packed(const float* packed_parts, int n_parts, int rows, int d_head, void* o,
                                float* lse, int dtype, void* stream) {
    if (!packed_parts || !o || n_parts <= 0 || rows <= 0) return FA_ERR_INVALID_ARGUMENT;
    if (d_head != 64 && d_head != 128) return FA_ERR_UNSUPPORTED;
    if (dtype != FA_DTYPE_F16 && dtype != FA_DTYPE_BF16) return FA_ERR_UNSUPPORTED;
    DeviceState* st = device_state();
    if (!st) return FA_ERR_CUDA;
    // [part][row][D + 1]: the merge reads the all-gather's receive buffer where it lies
    const long long w = d_head + 1;
    CombineOut out;
    out.o = o; out.lse = lse;
    return launch_combine(packed_parts, packed_parts + d_head, n_parts, (long long)rows * w, w, (long long)rows * w, w,
                          rows, d_head, out, dtype, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------
// KV-sequence-sharded decode: the local partial, the one all-gather and the merge
// behind one call.  NCCL is reached through dlopen so that the library has no
// link-time dependency on it (a process that never shards never loads it).
// ---------------------------------------------------------------------------
namespace fa {
namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*get_unique_id)(ncclUniqueId*) = nullptr;
    ncclResult_t (*comm_init_rank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*comm_destroy)(ncclComm_t) = nullptr;
    ncclResult_t (*comm_count)(const ncclComm_t, int*) = nullptr;
    ncclResult_t (*comm_user_rank)(const ncclComm_t, int*) = nullptr;
    ncclResult_t (*all_gather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*get_error_string)(ncclResult_t) = nullptr;
};
NcclApi g_nccl;
std::once_flag g_nccl_once;

// The NCCL already in the process (torch brings its own) or the system one.
const NcclApi* nccl_api() {
    std::call_once(g_nccl_once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return;
        NcclApi api;
        api.handle = h;
        api.get_unique_id = reinterpret_cast<decltype(api.get_unique_id)>(dlsym(h, "ncclGetUniqueId"));
        api.comm_init_rank = reinterpret_cast<decltype(api.comm_init_rank)>(dlsym(h, "ncclCommInitRank"));
        api.comm_destroy = reinterpret_cast<decltype(api.comm_destroy)>(dlsym(h, "ncclCommDestroy"));
        api.comm_count = reinterpret_cast<decltype(api.comm_count)>(dlsym(h, "ncclCommCount"));
        api.comm_user_rank = reinterpret_cast<decltype(api.comm_user_rank)>(dlsym(h, "ncclCommUserRank"));
        api.all_gather = reinterpret_cast<decltype(api.all_gather)>(dlsym(h, "ncclAllGather"));
        api.get_error_string = reinterpret_cast<decltype(api.get_error_string)>(dlsym(h, "ncclGetErrorString"));
        if (api.get_unique_id && api.comm_init_rank && api.comm_destroy && api.comm_count && api.comm_user_rank &&
            api.all_gather)
            g_nccl = api;
    });
    return g_nccl.handle ? &g_nccl : nullptr;
}

int note_nccl_error(const NcclApi* api, ncclResult_t r, const char* where) {
    char msg[200];
    snprintf(msg, sizeof(msg), "%s: NCCL %s", where,
             api && api->get_error_string ? api->get_error_string(r) : "error");
    return note_message(msg, FA_ERR_NCCL);
}

}  // namespace
}  // namespace fa

FA_EXPORT int fa_nccl_unique_id(void* id_out, size_t id_bytes) {
    if (!id_out || id_bytes < sizeof(ncclUniqueId)) return FA_ERR_INVALID_ARGUMENT;
    const NcclApi* api = nccl_api();
    if (!api) return note_message("libnccl.so.2 not found", FA_ERR_NCCL);
    ncclUniqueId id;
    ncclResult_t r = api->get_unique_id(&id);
    if (r != ncclSuccess) return note_nccl_error(api, r, "ncclGetUniqueId");
    memcpy(id_out, &id, sizeof(id));
    return FA_OK;
}

FA_EXPORT int fa_nccl_comm_create(void** comm_out, int n_ranks, const void* id, size_t id_bytes, int rank) {
    if (!comm_out || !id || id_bytes < sizeof(ncclUniqueId) || n_ranks <= 0 || rank < 0 || rank >= n_ranks)
        return FA_ERR_INVALID_ARGUMENT;
    const NcclApi* api = nccl_api();
    if (!api) return note_message("libnccl.so.2 not found", FA_ERR_NCCL);
    ncclUniqueId uid;
    memcpy(&uid, id, sizeof(uid));
    ncclComm_t comm = nullptr;
    ncclResult_t r = api->comm_init_rank(&comm, n_ranks, uid, rank);
    if (r != ncclSuccess) return note_nccl_error(api, r, "ncclCommInitRank");
    *comm_out = comm;
    return FA_OK;
}

FA_EXPORT int fa_nccl_comm_destroy(void* comm) {
    if (!comm) return FA_OK;
    const NcclApi* api = nccl_api();
    if (!api) return note_message("libnccl.so.2 not found", FA_ERR_NCCL);
    ncclResult_t r = api->comm_destroy(static_cast<ncclComm_t>(comm));
    return r == ncclSuccess ? FA_OK : note_nccl_error(api, r, "ncclCommDestroy");
}

FA_EXPORT size_t fa_decode_kv_sharded_gather_bytes(int batch_size, int num_heads, int d_head, int n_ranks) {
    if (batch_size <= 0 || num_heads <= 0 || d_head <= 0 || n_ranks <= 0) return 0;
    return (size_t)n_ranks * batch_size * num_heads * (d_head + 1) * sizeof(float);
}

FA_EXPORT int fa_decode_kv_sharded(const fa_decode_args* a, void* nccl_comm, float* gather, size_t gather_bytes) {
    if (!a || !nccl_comm || !gather || !a->o) return FA_ERR_INVALID_ARGUMENT;
    const bool no_keys = a->seq_len_kv == 0;              // this rank's slice of the cache is empty
    fa_decode_args local = *a;
    if (no_keys) { local.seq_len_kv = 1; if (!local.k) local.k = a->q; if (!local.v) local.v = a->q; }
    int rc = validate_decode(&local, false);
    if (rc != FA_OK) return rc;
    const NcclApi* api = nccl_api();
    if (!api) return note_message("libnccl.so.2 not found", FA_ERR_NCCL);
    DeviceState* st = device_state();
    if (!st) return FA_ERR_CUDA;
    if (st->cc_major != 10) return FA_ERR_NOT_SM100;
    ncclComm_t comm = static_cast<ncclComm_t>(nccl_comm);
    int n_ranks = 0, rank = 0;
    ncclResult_t r = api->comm_count(comm, &n_ranks);
    if (r == ncclSuccess) r = api->comm_user_rank(comm, &rank);
    if (r != ncclSuccess) return note_nccl_error(api, r, "ncclCommCount");
    const int rows = a->batch_size * a->num_heads;
    const size_t per_rank = (size_t)rows * (a->d_head + 1);
    if (gather_bytes < fa_decode_kv_sharded_gather_bytes(a->batch_size, a->num_heads, a->d_head, n_ranks) ||
        !aligned16(gather))
        return FA_ERR_WORKSPACE;
    cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
    float* mine = gather + (size_t)rank * per_rank;       // this rank's rows of the receive buffer
    if (no_keys) {
        empty_partial_kernel<<<rows, a->d_head, 0, stream>>>(mine, a->d_head);
        FA_CUDA_TRY(cudaGetLastError());
    } else {
        int splits, kps;
        plan_splits(a, st->sm_count, &splits, &kps);
        const size_t need = fa_decode_workspace_bytes(a->batch_size, a->num_heads, a->d_head, splits);
        if (!a->workspace || a->workspace_bytes < need || !aligned16(a->workspace)) return FA_ERR_WORKSPACE;
        // the merge of the local splits writes this rank's packed rows straight into the receive buffer
        CombineOut out;
        out.o_f32 = mine; out.o_f32_stride = a->d_head + 1;
        out.lse = mine + a->d_head; out.lse_stride = a->d_head + 1;
        if ((rc = decode_into(a, splits, kps, a->workspace, out)) != FA_OK) return rc;
    }
    // in place: the send buffer is this rank's block of the receive buffer
    r = api->all_gather(mine, gather, per_rank, ncclFloat, comm, stream);
    if (r != ncclSuccess) return note_nccl_error(api, r, "ncclAllGather");
    return fa_combine_packed(gather, n_ranks, rows, a->d_head, a->o, a->lse, a->dtype, a->stream);
}
