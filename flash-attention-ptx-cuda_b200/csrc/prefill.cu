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
// One CTA (8 warps) owns one 128-row query tile of one (batch, head):
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
#include "tmem_ld.cuh"

namespace fa {
namespace {

constexpr int kBM = 128;                 // query rows per CTA
constexpr int kThreads = 256;            // warps 0-3 softmax, 4 TMA, 5 MMA, 6-7 only donate registers
constexpr int kRegsSoftmax = 208;        // setmaxnreg targets: 128 * (208 + 48) = 256 * 128
constexpr int kRegsOther = 48;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;   // log2 units: rescale only if max grew > 2^8

// Barrier ids reported in the status word when a wait gives up.
enum : int { kBarQ = 1, kBarKFull = 2, kBarKEmpty = 3, kBarVFull = 4, kBarVEmpty = 5,
             kBarSFull = 6, kBarPFull = 7, kBarOFull = 8, kBarSFree = 9 };

// Packed pairs of fp32 (sm_100 has two-wide fp32 FMA/ADD on 64-bit register pairs).
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

#ifdef FA_PHASE_TIMING
// Development aid (not compiled into the shipped library): per-tile clock stamps of one CTA.
__device__ long long g_phase_ts[2][64][8];
__device__ long long g_cta_ts[4096][8];
#define FA_CTS(k) do { if (blockIdx.x < 4096) { g_cta_ts[blockIdx.x][k] = clock64(); } } while (0)
#define FA_TS(who, j, k) do { if (blockIdx.x == FA_PHASE_TIMING && (j) < 64) g_phase_ts[who][j][k] = clock64(); } while (0)
#else
#define FA_TS(who, j, k) do {} while (0)
#define FA_CTS(k) do {} while (0)
#endif

template <int D, int BN, int NK, int NV, bool FP8>
struct PrefillSmem {
    static constexpr int kNBox      = D / 64;              // 64-column (128-byte) boxes per 16-bit row
    static constexpr int kQBoxBytes = kBM * 128;
    static constexpr int kKVBoxBytes = BN * 128;
    // e4m3 rows of d_head 128 are exactly one 128-byte box.
    static constexpr int kQBytes    = FP8 ? kQBoxBytes : kNBox * kQBoxBytes;
    static constexpr int kKBytes    = FP8 ? kKVBoxBytes : kNBox * kKVBoxBytes;
    static constexpr int kVBytes    = kNBox * kKVBoxBytes; // 16-bit V operand of P V (e4m3: converted copy)
    static constexpr int kV8Bytes   = FP8 ? kKVBoxBytes : 0;   // landing buffer of the e4m3 V tile
    static constexpr int kTotal     = kQBytes + NK * kKBytes + NV * kVBytes + kV8Bytes + 1024;
};

// Two e4m3 codes -> two fp16 values (exact).
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint16_t v) {
    uint32_t r;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
    return r;
}

// FP8: Q, K, V are e4m3 codes with per-head scales.  S = Q K^T runs on the 8-bit tensor-core
// kind; V is converted e4m3 -> fp16 in shared memory by warps 6-7 (exact) and P V runs on the
// 16-bit kind with P in fp16, because an e4m3 P (3 mantissa bits) misses the output tolerance.
// The Q and K scales fold into the softmax scale, the V scale into the final normalisation;
// the output is bf16.
template <int D, int BN, int NK, int NV, bool CAUSAL, bool BF16, bool FP8>
__global__ void __launch_bounds__(kThreads, 2)
prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
               float* __restrict__ lse_out, int seq_len, int n_bh, int n_qtiles, float scale_log2_in,
               const float* __restrict__ q_scale, const float* __restrict__ k_scale,
               const float* __restrict__ v_scale, int* status) {
    static_assert(BN == 128, "the softmax warps hold one full 128-column score row in registers");
    static_assert(!FP8 || (D == 128 && NV == 1 && BF16), "e4m3 variant: d_head 128, bf16 output");
    using L = PrefillSmem<D, BN, NK, NV, FP8>;
    constexpr int NBOX = L::kNBox;
    constexpr uint32_t S_COL = 0;
    constexpr uint32_t O_COL = 128;
    // D = 64: P has its own columns, so S is free as soon as the softmax warps hold it in
    // registers and the next Q K^T can be issued before P V.  D = 128: P reuses the S columns.
    constexpr bool EARLY_QK = (D == 64);
    constexpr bool P_BF16 = BF16 && !FP8;                 // type of P (and of the V operand of P V)
    constexpr uint32_t P_COL = EARLY_QK ? 192 : 0;
    constexpr uint32_t TMEM_COLS = 256;
    constexpr uint32_t FMT = P_BF16 ? kFmtBF16 : kFmtF16;

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_q, bar_s, bar_p, bar_o, bar_sfree;
    __shared__ __align__(8) uint64_t bar_kf[NK], bar_ke[NK], bar_vf[NV], bar_ve[NV];
    __shared__ __align__(8) uint64_t bar_v8f, bar_v8e;    // e4m3 V landing buffer: filled / drained
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_s = base;
    const uint32_t k_s = q_s + L::kQBytes;
    const uint32_t v_s = k_s + NK * L::kKBytes;
    const uint32_t v8_s = v_s + NV * L::kVBytes;
    const uint32_t o_stage = FP8 ? v_s : q_s;             // epilogue staging: a dead operand buffer
    WaitCtl ctl{&abort_flag, status};

    // Heaviest query tiles first under the causal mask.
    const int work = blockIdx.x;
    const int qt = CAUSAL ? (n_qtiles - 1 - work / n_bh) : (work / n_bh);
    const int bh = work % n_bh;
    const int q_start = qt * kBM;
    const int kv_len = CAUSAL ? min(seq_len, q_start + kBM) : seq_len;
    const int n_kv = (kv_len + BN - 1) / BN;

#ifdef FA_PHASE_TIMING
    if (tid == 0 && blockIdx.x < 4096) {
        unsigned smid; asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
        g_cta_ts[blockIdx.x][6] = smid;
        g_cta_ts[blockIdx.x][7] = (long long)global_timer_ns();
    }
#endif
    if (tid == 0) FA_CTS(0);
    if (tid == 0) {
        mbar_init(smem_u32(&bar_q), 1);
        mbar_init(smem_u32(&bar_s), 1);
        mbar_init(smem_u32(&bar_p), 4);          // one arrival per softmax warp
        mbar_init(smem_u32(&bar_sfree), 4);
        mbar_init(smem_u32(&bar_o), 1);
        for (int i = 0; i < NK; i++) { mbar_init(smem_u32(&bar_kf[i]), 1); mbar_init(smem_u32(&bar_ke[i]), 1); }
        for (int i = 0; i < NV; i++) { mbar_init(smem_u32(&bar_vf[i]), FP8 ? 64 : 1); mbar_init(smem_u32(&bar_ve[i]), 1); }
        mbar_init(smem_u32(&bar_v8f), 1);
        mbar_init(smem_u32(&bar_v8e), 64);
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
    if (tid == 0) FA_CTS(1);

    if (warp >= 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
        if (warp == 4 && lane == 0) {
            // -------------------------------------------------------- TMA producer
            constexpr int NLOAD = FP8 ? 1 : NBOX;         // boxes per Q / K tile
            constexpr int XSTEP = FP8 ? 128 : 64;         // elements per box row
            mbar_arrive_expect_tx(smem_u32(&bar_q), L::kQBytes);
            for (int b = 0; b < NLOAD; b++)
                tma_load_3d(q_s + b * L::kQBoxBytes, &tm_q, smem_u32(&bar_q), b * XSTEP, q_start, bh);
            for (int j = 0; j < n_kv; j++) {
                const int sk = j % NK, sv = j % NV;
                if (j >= NK && !mbar_wait(smem_u32(&bar_ke[sk]), ((j / NK) - 1) & 1, ctl, kBarKEmpty)) break;
                mbar_arrive_expect_tx(smem_u32(&bar_kf[sk]), L::kKBytes);
                for (int b = 0; b < NLOAD; b++)
                    tma_load_3d(k_s + sk * L::kKBytes + b * L::kKVBoxBytes, &tm_k,
                                smem_u32(&bar_kf[sk]), b * XSTEP, j * BN, bh);
                if constexpr (FP8) {
                    // e4m3 V lands in its own buffer; warps 6-7 turn it into the fp16 operand.
                    if (j >= 1 && !mbar_wait(smem_u32(&bar_v8e), (j - 1) & 1, ctl, kBarVEmpty)) break;
                    mbar_arrive_expect_tx(smem_u32(&bar_v8f), L::kV8Bytes);
                    tma_load_3d(v8_s, &tm_v, smem_u32(&bar_v8f), 0, j * BN, bh);
                } else {
                    if (j >= NV && !mbar_wait(smem_u32(&bar_ve[sv]), ((j / NV) - 1) & 1, ctl, kBarVEmpty)) break;
                    mbar_arrive_expect_tx(smem_u32(&bar_vf[sv]), L::kVBytes);
                    for (int b = 0; b < NBOX; b++)
                        tma_load_3d(v_s + sv * L::kVBytes + b * L::kKVBoxBytes, &tm_v,
                                    smem_u32(&bar_vf[sv]), b * 64, j * BN, bh);
                }
            }
        } else if (warp == 5 && lane == 0) {
            // -------------------------------------------------------- MMA issuer
            constexpr uint32_t QKFMT = FP8 ? kFmtE4M3 : FMT;
            constexpr uint32_t idesc_qk = make_idesc(kBM, BN, QKFMT, QKFMT, kMajorK, kMajorK);
            constexpr uint32_t idesc_pv = make_idesc(kBM, D, FMT, FMT, kMajorK, kMajorMN);
            constexpr uint64_t hi_k = make_sdesc_hi(16, 1024);
            constexpr uint64_t hi_v = make_sdesc_hi(L::kKVBoxBytes, 1024);
            auto issue_qk = [&](int j) -> bool {
                const int sk = j % NK;
                if (!mbar_wait(smem_u32(&bar_kf[sk]), (j / NK) & 1, ctl, kBarKFull)) return false;
                if (EARLY_QK && j > 0 &&
                    !mbar_wait(smem_u32(&bar_sfree), (j - 1) & 1, ctl, kBarSFree)) return false;
                tc_fence_after();
                FA_TS(1, j, 0);
                const uint32_t kb = k_s + sk * L::kKBytes;
                if constexpr (FP8) {
#pragma unroll
                    for (int kk = 0; kk < D / 32; kk++)        // 32 e4m3 (32 bytes) of d_head per MMA
                        mma_f8_ss(tmem + S_COL, make_sdesc(q_s + kk * 32, hi_k), make_sdesc(kb + kk * 32, hi_k),
                                  idesc_qk, kk > 0);
                } else {
#pragma unroll
                    for (int kk = 0; kk < D / 16; kk++) {
                        const uint32_t qo = (kk >> 2) * L::kQBoxBytes + (kk & 3) * 32;
                        const uint32_t ko = (kk >> 2) * L::kKVBoxBytes + (kk & 3) * 32;
                        mma_f16_ss(tmem + S_COL, make_sdesc(q_s + qo, hi_k), make_sdesc(kb + ko, hi_k),
                                   idesc_qk, kk > 0);
                    }
                }
                tc_commit(smem_u32(&bar_s));
                tc_commit(smem_u32(&bar_ke[sk]));
                FA_TS(1, j, 1);
                return true;
            };
            auto issue_pv = [&](int j) -> bool {
                const int sv = j % NV;
                if (!mbar_wait(smem_u32(&bar_vf[sv]), (j / NV) & 1, ctl, kBarVFull)) return false;
                if (!mbar_wait(smem_u32(&bar_p), j & 1, ctl, kBarPFull)) return false;
                tc_fence_after();
                FA_TS(1, j, 2);
                const uint32_t vb = v_s + sv * L::kVBytes;
#pragma unroll
                for (int kk = 0; kk < BN / 16; kk++)
                    mma_f16_ts(tmem + O_COL, tmem + P_COL + kk * 8, make_sdesc(vb + kk * 2048, hi_v),
                               idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                tc_commit(smem_u32(&bar_o));
                tc_commit(smem_u32(&bar_ve[sv]));
                FA_TS(1, j, 3);
                return true;
            };
            bool ok = mbar_wait(smem_u32(&bar_q), 0, ctl, kBarQ);
            if (EARLY_QK) {
                // S(j+1) is computed while the softmax warps still work on S(j).
                ok = ok && issue_qk(0);
                for (int j = 0; ok && j < n_kv; j++) {
                    if (j + 1 < n_kv) ok = issue_qk(j + 1);
                    ok = ok && issue_pv(j);
                }
            } else {
                for (int j = 0; ok && j < n_kv; j++) ok = issue_qk(j) && issue_pv(j);
            }
        } else if (FP8 && warp >= 6) {
            // -------------------------------------------------------- e4m3 -> fp16 V converter
            const int ct = tid - 192;                     // 0..63
            for (int j = 0; j < n_kv; j++) {
                bool w = mbar_wait(smem_u32(&bar_v8f), j & 1, ctl, kBarVFull);
                // the fp16 copy of tile j-1 must have been consumed by P V(j-1)
                if (j >= 1) w = w && mbar_wait(smem_u32(&bar_ve[0]), (j - 1) & 1, ctl, kBarVEmpty);
                if (!__all_sync(0xffffffffu, w)) break;
#pragma unroll 4
                for (int it = 0; it < (BN * 16) / 64; it++) {
                    const int g = ct + it * 64;           // 8-element group: row g/16, group-in-row g%16
                    const int r = g >> 4, c8 = g & 15;
                    const uint32_t src = v8_s + r * 128 + ((((c8 >> 1) ^ (r & 7))) << 4) + ((c8 & 1) << 3);
                    uint32_t lo, hi;
                    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "r"(src));
                    const uint32_t w0 = e4m3x2_to_f16x2(static_cast<uint16_t>(lo & 0xFFFFu));
                    const uint32_t w1 = e4m3x2_to_f16x2(static_cast<uint16_t>(lo >> 16));
                    const uint32_t w2 = e4m3x2_to_f16x2(static_cast<uint16_t>(hi & 0xFFFFu));
                    const uint32_t w3 = e4m3x2_to_f16x2(static_cast<uint16_t>(hi >> 16));
                    const uint32_t dst = v_s + (c8 >> 3) * L::kKVBoxBytes + r * 128 + (((c8 & 7) ^ (r & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w0), "r"(w1),
                                 "r"(w2), "r"(w3) : "memory");
                }
                fence_proxy_async_smem();                 // the tensor core reads the copy through the async proxy
                mbar_arrive(smem_u32(&bar_vf[0]));
                mbar_arrive(smem_u32(&bar_v8e));
            }
        }
        __syncwarp();
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
        // ------------------------------------------------------------ softmax + epilogue
        const int r_in_tile = tid;                       // 0..127 == TMEM lane
        const int row = q_start + r_in_tile;
        const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
        const uint32_t t_s = tmem + lane_off + S_COL;
        const uint32_t t_p = tmem + lane_off + P_COL;
        const uint32_t t_o = tmem + lane_off + O_COL;
        const int row_limit = CAUSAL ? min(seq_len, row + 1) : seq_len;   // keys [0,row_limit) visible
        const int tile_min_limit = CAUSAL ? min(seq_len, q_start + 1) : seq_len;
        float scale_log2 = scale_log2_in;
        float out_scale = 1.0f;
        if constexpr (FP8) {
            scale_log2 *= q_scale[bh] * k_scale[bh];
            out_scale = v_scale[bh];
        }
        const uint64_t scale2 = pack2(scale_log2, scale_log2);
        float m_used = 0.0f;
        uint64_t lsum2 = pack2(0.0f, 0.0f);              // running row sum, two partial lanes
        bool ok = true;

        for (int j = 0; j < n_kv; j++) {
            const int kv_start = j * BN;
            // The votes keep the warp together: every lane leaves the loop or none does.
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_s), j & 1, ctl, kBarSFull))) { ok = false; break; }
            tc_fence_after();
            if (tid == 0) FA_TS(0, j, 0);
            if (tid == 0 && j == 0) FA_CTS(2);
            uint32_t s[128];
            tmem_ld128_wait(t_s, s);
            if (tid == 0) FA_TS(0, j, 1);
            if (EARLY_QK) {                              // S is in registers: release the TMEM columns
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar_sfree));
            }
            if ((tile_min_limit - kv_start) < BN) {      // tile touches the mask or the ragged end
                const int limit = row_limit - kv_start;  // columns [0,limit) are visible
#pragma unroll
                for (int i = 0; i < 128; i++) s[i] = (i < limit) ? s[i] : 0xff800000u;   // -inf
            }
            // ---- row maximum of the raw scores
            float a0 = -INFINITY, a1 = -INFINITY, a2 = -INFINITY, a3 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 128; i += 8) {
                a0 = max3(a0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
                a1 = max3(a1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
                a2 = max3(a2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
                a3 = max3(a3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
            }
            const float tile_max = fmaxf(max3(a0, a1, a2), a3) * scale_log2;
            if (tid == 0) FA_TS(0, j, 2);
            bool need = false;
            if (j == 0) m_used = tile_max;
            else need = tile_max > m_used + kRescaleThreshold;

            // ---- rare: the running max grew by more than the threshold -> rescale O in TMEM.
            // O(j-1) must be complete first.  D = 128: S(j) complete implies P V(j-1) complete
            // (the tensor pipe runs in order); D = 64: Q K^T(j) was issued ahead of P V(j-1),
            // so wait for its commit.
            bool pv_prev_done = !(EARLY_QK && j > 0);
            if (__any_sync(0xffffffffu, need)) {
                if (!pv_prev_done) {
                    if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_o), (j - 1) & 1, ctl, kBarOFull))) { ok = false; break; }
                    tc_fence_after();
                    pv_prev_done = true;
                }
                float factor = 1.0f;
                if (need) {
                    factor = ex2_approx(m_used - tile_max);
                    m_used = tile_max;
                    lsum2 = fma2(lsum2, pack2(factor, factor), pack2(0.0f, 0.0f));
                }
#pragma unroll 1
                for (int c = 0; c < D / 32; c++) {
                    uint32_t t[32];
                    tmem_ld32_wait(t_o + c * 32, t);
#pragma unroll
                    for (int i = 0; i < 32; i++) t[i] = __float_as_uint(__uint_as_float(t[i]) * factor);
                    tmem_st_x32(t_o + c * 32, t);
                }
                tmem_wait_st();
            }

            if (tid == 0) FA_TS(0, j, 3);
            // ---- p = 2^(s*scale*log2e - m); row sum; P as packed 16-bit pairs, kept in
            // registers (they replace the scores two for one) until the P columns are free.
            const uint64_t negm2 = pack2(-m_used, -m_used);
            uint32_t pk[64];
#pragma unroll
            for (int i = 0; i < 64; i++) {
                const uint64_t t = fma2(pack2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1])), scale2, negm2);
                float t0, t1;
                unpack2(t, t0, t1);
                const float p0 = ex2_approx(t0), p1 = ex2_approx(t1);
                lsum2 = add2(lsum2, pack2(p0, p1));
                pk[i] = pack_16<P_BF16>(p0, p1);
            }
            if (!pv_prev_done) {
                // P(j-1) must have been consumed by P V(j-1) before it is overwritten; by now it
                // normally has been, so this wait rarely blocks.
                if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_o), (j - 1) & 1, ctl, kBarOFull))) { ok = false; break; }
                tc_fence_after();
            }
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t (&chunk)[16] = *reinterpret_cast<uint32_t (*)[16]>(&pk[c * 16]);
                tmem_st_x16(t_p + c * 16, chunk);
            }
            if (tid == 0) FA_TS(0, j, 4);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_p));
            if (tid == 0) FA_TS(0, j, 5);
        }

        if (tid == 0) FA_CTS(3);
        // ---- epilogue: O / l -> 16-bit -> swizzled staging (the Q buffer) -> TMA store
        ok = __all_sync(0xffffffffu, ok && mbar_wait(smem_u32(&bar_o), (n_kv - 1) & 1, ctl, kBarOFull));
        tc_fence_after();
        if (ok) {
            float l0, l1;
            unpack2(lsum2, l0, l1);
            const float l_run = l0 + l1;
            const float inv_l = out_scale / l_run;
#pragma unroll 1
            for (int c = 0; c < D / 32; c++) {
                uint32_t t[32];
                tmem_ld32_wait(t_o + c * 32, t);
#pragma unroll
                for (int g4 = 0; g4 < 4; g4++) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; e++)
                        w[e] = pack_16<BF16>(__uint_as_float(t[g4 * 8 + 2 * e]) * inv_l,
                                             __uint_as_float(t[g4 * 8 + 2 * e + 1]) * inv_l);
                    const int g = c * 4 + g4;             // 8-element (16-byte) group index in the row
                    const uint32_t addr = o_stage + (g >> 3) * L::kQBoxBytes + r_in_tile * 128 +
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
                tma_store_3d(&tm_o, o_stage + b * L::kQBoxBytes, b * 64, q_start, bh);
            tma_store_commit();
            tma_store_wait_read();        // the CTA may exit once the staging buffer has been read
        }
        if (tid == 0) FA_CTS(4);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 5) tmem_dealloc(tmem, TMEM_COLS);
}

template <int D, int BN, int NK, int NV, bool CAUSAL, bool BF16, bool FP8 = false>
int launch_instance(const fa_prefill_args& a, DeviceState* st, const CUtensorMap& tq,
                    const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to) {
    using L = PrefillSmem<D, BN, NK, NV, FP8>;
    auto kernel = prefill_kernel<D, BN, NK, NV, CAUSAL, BF16, FP8>;
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
        tq, tk, tv, to, a.lse, a.seq_len, n_bh, n_qtiles, a.scale * kLog2e, a.q_scale, a.k_scale,
        a.v_scale, st->status);
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

#ifdef FA_PHASE_TIMING
extern "C" __attribute__((visibility("default"))) int fa_debug_phase_ts(long long* out) {
    return (int)cudaMemcpyFromSymbol(out, g_phase_ts, sizeof(long long) * 2 * 64 * 8);
}
extern "C" __attribute__((visibility("default"))) int fa_debug_cta_ts(long long* out) {
    return (int)cudaMemcpyFromSymbol(out, g_cta_ts, sizeof(long long) * 4096 * 8);
}
#endif

// e4m3 inputs (d_head 128), bf16 output.
int launch_prefill_fp8(const fa_prefill_args& a, DeviceState* st) {
    const uint64_t n_bh = (uint64_t)a.batch_size * a.num_heads;
    constexpr int BN = 128;
    CUtensorMap tq, tk, tv, to;
    int rc;
    if ((rc = make_tensor_map_3d(&tq, a.q, FA_DTYPE_E4M3, 128, a.seq_len, n_bh, 128, kBM)) != FA_OK) return rc;
    if ((rc = make_tensor_map_3d(&tk, a.k, FA_DTYPE_E4M3, 128, a.seq_len, n_bh, 128, BN)) != FA_OK) return rc;
    if ((rc = make_tensor_map_3d(&tv, a.v, FA_DTYPE_E4M3, 128, a.seq_len, n_bh, 128, BN)) != FA_OK) return rc;
    if ((rc = make_tensor_map_3d(&to, a.o, FA_DTYPE_BF16, 128, a.seq_len, n_bh, 64, kBM)) != FA_OK) return rc;
    if (a.causal) return launch_instance<128, BN, 2, 1, true, true, true>(a, st, tq, tk, tv, to);
    return launch_instance<128, BN, 2, 1, false, true, true>(a, st, tq, tk, tv, to);
}

}  // namespace fa
