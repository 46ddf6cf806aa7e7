// Prefill forward kernel for sm_100a, 16-bit inputs (fp16 / bf16), d_head 64 or
// 128, causal or not, any sequence length.
//
// Replaces the reference's kernel and launcher
// (kernels/flash_attention.cu:116-507 flash_attention_ptx_kernel, :534-579
// launch_variant, :595-617 launch_flash_attention).  Same mathematics - per query
// row an online softmax over key tiles with a running max and sum, O += P V,
// final O / sum and LSE = max + log(sum) (:303-314 scale and mask, :332-401
// softmax, :411-425 rescale, :437-468 P V, :476-505 epilogue) - but none of its
// structure: no mma.sync, no ldmatrix, no cp.async, no block-wide barriers in
// the loop.
//
// One CTA owns one 128-row query tile of one (batch, head):
//   warp 4 (one lane)  TMA producer: Q once, then K and V tiles through two
//                      mbarrier-guarded shared-memory rings (128-byte swizzle);
//   warp 5 (one lane)  issues tcgen05.mma: S = Q K^T into TMEM, later
//                      O += P V with P read from TMEM and V (MN-major) from
//                      shared memory; completion is signalled by tcgen05.commit;
//   warps 0-3          softmax: thread t owns query row t (TMEM lane t), reads
//                      its S row with tcgen05.ld, keeps the running max / sum in
//                      registers (no cross-thread reduction), writes P as packed
//                      16-bit pairs with tcgen05.st, rescales O in TMEM only when
//                      the max grew by more than 2^8, and in the epilogue
//                      normalises O, stages it in swizzled shared memory and
//                      stores it with one TMA store per 64 columns; LSE rows are
//                      written as coalesced fp32.
// Two CTAs fit on an SM (TMEM: 256 of 512 columns each), so one CTA's softmax
// overlaps the other's tensor-core work.
#include <cmath>

#include "host_common.h"
#include "ptx.cuh"

namespace fa {
namespace {

constexpr int kBM = 128;                 // query rows per CTA
constexpr int kThreads = 192;            // 4 softmax warps + TMA warp + MMA warp
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;   // log2 units: rescale only if max grew > 2^8

// Barrier ids reported in the status word when a wait gives up.
enum : int { kBarQ = 1, kBarKFull = 2, kBarKEmpty = 3, kBarVFull = 4, kBarVEmpty = 5,
             kBarSFull = 6, kBarPFull = 7, kBarOFull = 8 };

__device__ __forceinline__ void tmem_wait_ld_tie(uint32_t (&r)[32]) {
    // Waits for outstanding tcgen05.ld and ties the destination registers to the
    // wait so that no use of them can be scheduled ahead of it.
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]),
                   "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]),
                   "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]),
                   "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                   "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]),
                   "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}

template <int D, int BN, int NK, int NV>
struct PrefillSmem {
    static constexpr int kNBox      = D / 64;              // 64-column (128-byte) boxes per row
    static constexpr int kQBoxBytes = kBM * 128;
    static constexpr int kKVBoxBytes = BN * 128;
    static constexpr int kQBytes    = kNBox * kQBoxBytes;
    static constexpr int kKVBytes   = kNBox * kKVBoxBytes;
    static constexpr int kTotal     = kQBytes + (NK + NV) * kKVBytes + 1024;   // + alignment slack
};

template <int D, int BN, int NK, int NV, bool CAUSAL, bool BF16>
__global__ void __launch_bounds__(kThreads, 2)
prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
               float* __restrict__ lse_out, int seq_len, int n_bh, int n_qtiles, float scale_log2,
               int* status) {
    using L = PrefillSmem<D, BN, NK, NV>;
    constexpr int NBOX = L::kNBox;
    constexpr int NCH  = BN / 32;                         // 32-column chunks of an S row
    constexpr uint32_t S_COL = 0;
    constexpr uint32_t O_COL = 128;
    constexpr uint32_t P_COL = (D == 64) ? 192 : 0;       // D = 128: P reuses the S columns it replaces
    constexpr uint32_t TMEM_COLS = 256;
    constexpr uint32_t FMT = BF16 ? kFmtBF16 : kFmtF16;

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_q, bar_s, bar_p, bar_o;
    __shared__ __align__(8) uint64_t bar_kf[NK], bar_ke[NK], bar_vf[NV], bar_ve[NV];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_s = base;
    const uint32_t k_s = q_s + L::kQBytes;
    const uint32_t v_s = k_s + NK * L::kKVBytes;
    WaitCtl ctl{&abort_flag, status};

    // Heaviest query tiles first under the causal mask.
    const int work = blockIdx.x;
    const int qt = CAUSAL ? (n_qtiles - 1 - work / n_bh) : (work / n_bh);
    const int bh = work % n_bh;
    const int q_start = qt * kBM;
    const int kv_len = CAUSAL ? min(seq_len, q_start + kBM) : seq_len;
    const int n_kv = (kv_len + BN - 1) / BN;

    if (tid == 0) {
        mbar_init(smem_u32(&bar_q), 1);
        mbar_init(smem_u32(&bar_s), 1);
        mbar_init(smem_u32(&bar_p), 128);
        mbar_init(smem_u32(&bar_o), 1);
        for (int i = 0; i < NK; i++) { mbar_init(smem_u32(&bar_kf[i]), 1); mbar_init(smem_u32(&bar_ke[i]), 1); }
        for (int i = 0; i < NV; i++) { mbar_init(smem_u32(&bar_vf[i]), 1); mbar_init(smem_u32(&bar_ve[i]), 1); }
        abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 4 && lane == 0) {
        prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v); prefetch_tensormap(&tm_o);
    }
    __syncthreads();
    if (warp == 5) tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    if (warp == 4) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(smem_u32(&bar_q), L::kQBytes);
            for (int b = 0; b < NBOX; b++)
                tma_load_3d(q_s + b * L::kQBoxBytes, &tm_q, smem_u32(&bar_q), b * 64, q_start, bh);
            for (int j = 0; j < n_kv; j++) {
                const int sk = j % NK, sv = j % NV;
                if (j >= NK && !mbar_wait(smem_u32(&bar_ke[sk]), ((j / NK) - 1) & 1, ctl, kBarKEmpty)) break;
                mbar_arrive_expect_tx(smem_u32(&bar_kf[sk]), L::kKVBytes);
                for (int b = 0; b < NBOX; b++)
                    tma_load_3d(k_s + sk * L::kKVBytes + b * L::kKVBoxBytes, &tm_k,
                                smem_u32(&bar_kf[sk]), b * 64, j * BN, bh);
                if (j >= NV && !mbar_wait(smem_u32(&bar_ve[sv]), ((j / NV) - 1) & 1, ctl, kBarVEmpty)) break;
                mbar_arrive_expect_tx(smem_u32(&bar_vf[sv]), L::kKVBytes);
                for (int b = 0; b < NBOX; b++)
                    tma_load_3d(v_s + sv * L::kKVBytes + b * L::kKVBoxBytes, &tm_v,
                                smem_u32(&bar_vf[sv]), b * 64, j * BN, bh);
            }
        }
        __syncwarp();
    } else if (warp == 5) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = make_idesc(kBM, BN, FMT, FMT, kMajorK, kMajorK);
            constexpr uint32_t idesc_pv = make_idesc(kBM, D, FMT, FMT, kMajorK, kMajorMN);
            constexpr uint64_t hi_k = make_sdesc_hi(16, 1024);
            constexpr uint64_t hi_v = make_sdesc_hi(L::kKVBoxBytes, 1024);
            bool ok = mbar_wait(smem_u32(&bar_q), 0, ctl, kBarQ);
            for (int j = 0; ok && j < n_kv; j++) {
                const int sk = j % NK, sv = j % NV;
                if (!mbar_wait(smem_u32(&bar_kf[sk]), (j / NK) & 1, ctl, kBarKFull)) break;
                tc_fence_after();
                const uint32_t kb = k_s + sk * L::kKVBytes;
#pragma unroll
                for (int kk = 0; kk < D / 16; kk++) {
                    const uint32_t qo = (kk >> 2) * L::kQBoxBytes + (kk & 3) * 32;
                    const uint32_t ko = (kk >> 2) * L::kKVBoxBytes + (kk & 3) * 32;
                    mma_f16_ss(tmem + S_COL, make_sdesc(q_s + qo, hi_k), make_sdesc(kb + ko, hi_k),
                               idesc_qk, kk > 0);
                }
                tc_commit(smem_u32(&bar_s));
                tc_commit(smem_u32(&bar_ke[sk]));
                if (!mbar_wait(smem_u32(&bar_vf[sv]), (j / NV) & 1, ctl, kBarVFull)) break;
                if (!mbar_wait(smem_u32(&bar_p), j & 1, ctl, kBarPFull)) break;
                tc_fence_after();
                const uint32_t vb = v_s + sv * L::kKVBytes;
#pragma unroll
                for (int kk = 0; kk < BN / 16; kk++)
                    mma_f16_ts(tmem + O_COL, tmem + P_COL + kk * 8, make_sdesc(vb + kk * 2048, hi_v),
                               idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                tc_commit(smem_u32(&bar_o));
                tc_commit(smem_u32(&bar_ve[sv]));
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ softmax + epilogue
        const int r_in_tile = tid;                       // 0..127 == TMEM lane
        const int row = q_start + r_in_tile;
        const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
        const uint32_t t_s = tmem + lane_off + S_COL;
        const uint32_t t_p = tmem + lane_off + P_COL;
        const uint32_t t_o = tmem + lane_off + O_COL;
        const int row_limit = CAUSAL ? min(seq_len, row + 1) : seq_len;   // keys [0,row_limit) visible
        const int tile_min_limit = CAUSAL ? min(seq_len, q_start + 1) : seq_len;
        float m_used = 0.0f, l_run = 0.0f;
        bool ok = true;

        for (int j = 0; j < n_kv; j++) {
            const int kv_start = j * BN;
            // The vote keeps the warp together: every lane leaves the loop or none does.
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_s), j & 1, ctl, kBarSFull))) { ok = false; break; }
            tc_fence_after();
            const bool masked_tile = (tile_min_limit - kv_start) < BN;
            const int limit = row_limit - kv_start;       // columns [0,limit) of this tile are visible

            uint32_t ra[32], rb[32];
            // ---- pass 1: row maximum of the raw scores
            float mx = -INFINITY;
            tmem_ld_x32(t_s, ra);
#pragma unroll
            for (int c = 0; c < NCH; c++) {
                uint32_t (&cur)[32] = (c & 1) ? rb : ra;
                uint32_t (&nxt)[32] = (c & 1) ? ra : rb;
                tmem_wait_ld_tie(cur);
                if (c + 1 < NCH) tmem_ld_x32(t_s + (c + 1) * 32, nxt);
                if (masked_tile) {
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        mx = fmaxf(mx, (c * 32 + i < limit) ? __uint_as_float(cur[i]) : -INFINITY);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) mx = fmaxf(mx, __uint_as_float(cur[i]));
                }
            }
            const float tile_max = mx * scale_log2;
            bool need = false;
            if (j == 0) m_used = tile_max;
            else need = tile_max > m_used + kRescaleThreshold;

            // ---- rare: the running max grew by more than the threshold -> rescale O in TMEM
            if (__any_sync(0xffffffffu, need)) {
                if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_o), (j - 1) & 1, ctl, kBarOFull))) { ok = false; break; }
                tc_fence_after();
                float factor = 1.0f;
                if (need) {
                    factor = ex2_approx(m_used - tile_max);
                    m_used = tile_max;
                    l_run *= factor;
                }
#pragma unroll 1
                for (int c = 0; c < D / 32; c++) {
                    tmem_ld_x32(t_o + c * 32, ra);
                    tmem_wait_ld_tie(ra);
#pragma unroll
                    for (int i = 0; i < 32; i++) ra[i] = __float_as_uint(__uint_as_float(ra[i]) * factor);
                    tmem_st_x32(t_o + c * 32, ra);
                }
                tmem_wait_st();
            }

            // ---- pass 2: p = 2^(s*scale*log2e - m); row sum; P -> TMEM as packed 16-bit
            const float neg_m = -m_used;
            float psum = 0.0f;
            tmem_ld_x32(t_s, ra);
#pragma unroll
            for (int c = 0; c < NCH; c++) {
                uint32_t (&cur)[32] = (c & 1) ? rb : ra;
                uint32_t (&nxt)[32] = (c & 1) ? ra : rb;
                tmem_wait_ld_tie(cur);
                if (c + 1 < NCH) tmem_ld_x32(t_s + (c + 1) * 32, nxt);
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float s0 = __uint_as_float(cur[i]), s1 = __uint_as_float(cur[i + 1]);
                    if (masked_tile) {
                        s0 = (c * 32 + i < limit) ? s0 : -INFINITY;
                        s1 = (c * 32 + i + 1 < limit) ? s1 : -INFINITY;
                    }
                    const float p0 = ex2_approx(fmaf(s0, scale_log2, neg_m));
                    const float p1 = ex2_approx(fmaf(s1, scale_log2, neg_m));
                    psum += p0 + p1;
                    pk[i >> 1] = pack_16<BF16>(p0, p1);
                }
                tmem_st_x16(t_p + c * 16, pk);
            }
            l_run += psum;
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(smem_u32(&bar_p));
        }

        // ---- epilogue: O / l -> 16-bit -> swizzled staging (the Q buffer) -> TMA store
        ok = __all_sync(0xffffffffu, ok && mbar_wait(smem_u32(&bar_o), (n_kv - 1) & 1, ctl, kBarOFull));
        tc_fence_after();
        if (ok) {
            const float inv_l = 1.0f / l_run;
            uint32_t ra[32];
#pragma unroll 1
            for (int c = 0; c < D / 32; c++) {
                tmem_ld_x32(t_o + c * 32, ra);
                tmem_wait_ld_tie(ra);
#pragma unroll
                for (int t = 0; t < 4; t++) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; e++)
                        w[e] = pack_16<BF16>(__uint_as_float(ra[t * 8 + 2 * e]) * inv_l,
                                             __uint_as_float(ra[t * 8 + 2 * e + 1]) * inv_l);
                    const int g = c * 4 + t;              // 8-element (16-byte) group index in the row
                    const uint32_t addr = q_s + (g >> 3) * L::kQBoxBytes + r_in_tile * 128 +
                                          (((g & 7) ^ (r_in_tile & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]),
                                 "r"(w[1]), "r"(w[2]), "r"(w[3])
                                 : "memory");
                }
            }
            if (lse_out != nullptr && row < seq_len)
                lse_out[static_cast<size_t>(bh) * seq_len + row] = kLn2 * (m_used + log2f(l_run));
        }
        fence_proxy_async_smem();
        named_barrier_sync(1, 128);
        if (ok && tid == 0) {
            for (int b = 0; b < NBOX; b++)
                tma_store_3d(&tm_o, q_s + b * L::kQBoxBytes, b * 64, q_start, bh);
            tma_store_commit();
            tma_store_wait_all();
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 5) tmem_dealloc(tmem, TMEM_COLS);
}

template <int D, int BN, int NK, int NV, bool CAUSAL, bool BF16>
int launch_instance(const fa_prefill_args& a, DeviceState* st, const CUtensorMap& tq,
                    const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to) {
    using L = PrefillSmem<D, BN, NK, NV>;
    auto kernel = prefill_kernel<D, BN, NK, NV, CAUSAL, BF16>;
    static bool configured[64] = {};
    if (!configured[st->device]) {
        FA_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
        configured[st->device] = true;
    }
    const int n_bh = a.batch_size * a.num_heads;
    const int n_qtiles = (a.seq_len + kBM - 1) / kBM;
    const long long n_cta = (long long)n_bh * n_qtiles;
    if (n_cta > 0x7FFFFFFFll) return FA_ERR_INVALID_ARGUMENT;
    kernel<<<(unsigned)n_cta, kThreads, L::kTotal, static_cast<cudaStream_t>(a.stream)>>>(
        tq, tk, tv, to, a.lse, a.seq_len, n_bh, n_qtiles, a.scale * kLog2e, st->status);
    FA_CUDA_TRY(cudaGetLastError());
    return FA_OK;
}

}  // namespace

int launch_prefill_16bit(const fa_prefill_args& a, DeviceState* st) {
    const uint64_t n_bh = (uint64_t)a.batch_size * a.num_heads;
    constexpr int BN = 128;
    CUtensorMap tq, tk, tv, to;
    int rc;
    if ((rc = make_tensor_map_3d(&tq, a.q, a.dtype, a.d_head, a.seq_len, n_bh, 64, kBM)) != FA_OK) return rc;
    if ((rc = make_tensor_map_3d(&tk, a.k, a.dtype, a.d_head, a.seq_len, n_bh, 64, BN)) != FA_OK) return rc;
    if ((rc = make_tensor_map_3d(&tv, a.v, a.dtype, a.d_head, a.seq_len, n_bh, 64, BN)) != FA_OK) return rc;
    if ((rc = make_tensor_map_3d(&to, a.o, a.dtype, a.d_head, a.seq_len, n_bh, 64, kBM)) != FA_OK) return rc;
    const bool bf = a.dtype == FA_DTYPE_BF16;
    const bool causal = a.causal != 0;
#define FA_DISPATCH(DH, NKS, NVS)                                                              \
    (causal ? (bf ? launch_instance<DH, BN, NKS, NVS, true, true>(a, st, tq, tk, tv, to)       \
                  : launch_instance<DH, BN, NKS, NVS, true, false>(a, st, tq, tk, tv, to))     \
            : (bf ? launch_instance<DH, BN, NKS, NVS, false, true>(a, st, tq, tk, tv, to)      \
                  : launch_instance<DH, BN, NKS, NVS, false, false>(a, st, tq, tk, tv, to)))
    if (a.d_head == 64) return FA_DISPATCH(64, 2, 2);
    return FA_DISPATCH(128, 1, 1);
#undef FA_DISPATCH
}

// Placeholder until the e4m3 kernel lands: reports the variant as not built.
int launch_prefill_fp8(const fa_prefill_args&, DeviceState*) { return FA_ERR_UNSUPPORTED; }

}  // namespace fa
