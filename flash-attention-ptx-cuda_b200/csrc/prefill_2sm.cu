// Prefill forward kernel for sm_100a on PAIRS of CTAs (thread-block clusters of two, tcgen05
// cta_group::2): fp16 / bf16, d_head 128, causal or not, any sequence length.
//
// Replaces the reference's kernel and launcher for long sequences at d_head 128
// (kernels/flash_attention.cu:116-507, :534-579; the reference's dispatcher, :595-617, likewise
// picks a tile variant by problem size).  Same mathematics (online softmax :332-401, rescale
// :411-425, O += P V :437-468, O / sum and LSE :476-505).
//
// Why pairs.  At d_head 128 the one-CTA kernel is bound by the K/V stream from L2 into shared
// memory (64 KB per 128-key tile per SM; with the loads compiled out it runs a third faster).
// Here the two CTAs of a cluster work on two adjacent 128-row query tiles of the same head and
// share every key tile: each CTA loads only HALF of it (K: 64 of the 128 keys; V: 64 of the 128
// head-dim columns) and one MMA instruction, issued by a thread of the even ("leader") CTA,
// covers both CTAs' query tiles (M = 256), reading the B operand's two halves from the two shared
// memories.  Per SM that halves the K/V traffic, the shared-memory footprint of a stage and the
// number of MMA instructions issued.  Every CTA fetches its own halves with plain tiled loads whose
// byte counts are credited to the leader's barrier; nothing is copied to more than one CTA.
//
// Inside a CTA the structure is the one-CTA kernel's: two softmax groups on alternate key tiles
// (one thread per query row, scores in registers, P written back over the scores in TMEM, the max
// in use handed from tile to tile through tagged shared-memory slots, O rescaled lazily in TMEM),
// epilogue warps, producers; three score buffers U0..U2 and O in TMEM.  What crosses CTAs:
//   leader <- peer : "my P is in TMEM" and "my epilogue has read O" (remote mbarrier arrivals;
//                    the leader's issuers wait for both CTAs), K / V / Q bytes landed (credited by
//                    the loads themselves);
//   leader -> both : every completion (Q K^T done, P V done, Q free, O done) is ONE commit that
//                    arrives on the same barrier in both CTAs.
// Under the causal mask the even tile of a pair walks one key tile fewer than the odd one; it sees
// that last tile fully masked (P = 0, max and sum untouched).
//
// Every wait is bounded; on expiry the CTA records (1 << 16) | barrier id in the device status
// word and every role leaves its loops; the peer then runs into its own limits.
#include <cmath>

#include "host_common.h"
#include "ptx.cuh"
#include "tmem_ld.cuh"

namespace fa {
namespace {

constexpr int kBM = 128;                 // query rows per CTA (256 per cluster)
constexpr int kBN = 128;                 // keys per tile
constexpr int kThreads = 512;
constexpr int kRegsLaunch = (65536 / kThreads) / 8 * 8;
constexpr int kRegsSoftmax = 192;        // warps 0-7
constexpr int kRegsOther = 64;           // warps 8-15
static_assert(256 * kRegsSoftmax + 256 * kRegsOther <= kThreads * kRegsLaunch,
              "setmaxnreg targets exceed the CTA's register pool");
constexpr int kNU = 3;                   // score buffers in TMEM (S, then P in place)
constexpr int kRing = 8;                 // entries of the completion rings (> stage counts)
constexpr int kStages = 4;               // K and V stages (half tiles of 16 KB)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;

// Barrier ids reported in the status word when a wait gives up (0x60 + ...: this kernel).
enum : int { k2QFull = 0x61, k2QFree, k2KFull, k2KFree, k2VFull, k2VFree, k2SFull, k2SFree, k2PFull, k2PV,
             k2OFree, k2ODone, k2M, k2Epi, k2Stats, k2StatsFree };

template <int D>
struct PairSmem2 {
    static_assert(D == 128, "the cluster kernel is built for d_head 128");
    static constexpr int kBox    = 128 * 128;            // 128 rows x 128 bytes
    static constexpr int kQBytes = 2 * kBox;             // this CTA's whole query tile
    static constexpr int kKHalf  = 2 * (64 * 128);       // 64 keys x 128 d: two boxes of 64 rows
    static constexpr int kVHalf  = kBox;                 // 128 keys x 64 d: one box
    static constexpr int kOBytes = 2 * kBox;
    static constexpr int kTotal  = kQBytes + kStages * (kKHalf + kVHalf) + kOBytes + 1024;
};

struct Item2 { int bh, pair, n_kv; };

// Work list over (pair of query tiles, head), heaviest first under the causal mask, dealt to the
// clusters in boustrophedon order; heads in groups so that the K/V in flight stay in L2.
template <bool CAUSAL>
__device__ __forceinline__ bool get_item2(int round, int n_items, int n_bh, int n_pairs, int seq_len,
                                          int heads_per_group, Item2& it) {
    const int G = gridDim.x >> 1, c = blockIdx.x >> 1;
    const int idx = (round & 1) ? round * G + (G - 1 - c) : round * G + c;
    if (idx >= n_items) return false;
    const int per_group = heads_per_group * n_pairs;
    const int gi = idx / per_group, rem = idx - gi * per_group;
    const int h0 = gi * heads_per_group, hin = min(heads_per_group, n_bh - h0);
    const int rank = rem / hin;
    it.bh = h0 + rem - rank * hin;
    it.pair = CAUSAL ? (n_pairs - 1 - rank) : rank;
    const int n_all = (seq_len + kBN - 1) / kBN;
    it.n_kv = CAUSAL ? min(n_all, 2 * it.pair + 2) : n_all;
    return true;
}

template <int D, bool CAUSAL, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
prefill_2sm_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                   float* __restrict__ lse_out, int seq_len, int n_bh, int n_pairs, int n_items,
                   int heads_per_group, float scale_log2, int* status) {
    using L = PairSmem2<D>;
    constexpr int NBOX = D / 64;
    constexpr uint32_t O_COL = kNU * 128;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t FMT = BF16 ? kFmtBF16 : kFmtF16;

    extern __shared__ uint8_t smem_raw[];
    // The same layout in both CTAs: remote arrivals and the leader's commits address a barrier
    // by its offset.
    __shared__ __align__(8) uint64_t bar_qf, bar_ofree;
    __shared__ __align__(8) uint64_t bar_kf[kStages], bar_vf[kStages];
    __shared__ __align__(8) uint64_t bar_qk[kRing], bar_pvd[kRing];      // completion rings (leader's commits, both CTAs)
    __shared__ __align__(8) uint64_t bar_pf[kNU];                         // leader: P of both CTAs is in TMEM
    __shared__ __align__(8) uint64_t bar_epi;
    __shared__ __align__(8) uint2 m_slot[2][128];
    __shared__ float xm[2][2][128], xsum[2][2][128];
    __shared__ __align__(8) uint64_t bar_stats[2], bar_stats_free[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_ctarank();              // 0 = leader (issues the pair's MMAs)
    const bool leader = rank == 0;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_s = base;
    const uint32_t k_s = q_s + L::kQBytes;
    const uint32_t v_s = k_s + kStages * L::kKHalf;
    const uint32_t o_s = v_s + kStages * L::kVHalf;
    WaitCtl ctl{&abort_flag, status};

    if (tid == 0) {
        mbar_init(smem_u32(&bar_qf), 1);
        mbar_init(smem_u32(&bar_ofree), 8);              // the epilogue warps of BOTH CTAs have read O
        for (int i = 0; i < kStages; i++) { mbar_init(smem_u32(&bar_kf[i]), 1); mbar_init(smem_u32(&bar_vf[i]), 1); }
        for (int i = 0; i < kRing; i++) { mbar_init(smem_u32(&bar_qk[i]), 1); mbar_init(smem_u32(&bar_pvd[i]), 1); }
        for (int i = 0; i < kNU; i++) mbar_init(smem_u32(&bar_pf[i]), 8);     // four warps of the owning group in each CTA
        mbar_init(smem_u32(&bar_epi), 4);
        for (int i = 0; i < 2; i++) { mbar_init(smem_u32(&bar_stats[i]), 8); mbar_init(smem_u32(&bar_stats_free[i]), 4); }
        abort_flag = 0;
        fence_mbar_init();
    }
    if (tid < 256) m_slot[tid >> 7][tid & 127] = make_uint2(0u, 0xFFFFFFFFu);
    if (warp == 8 && lane == 0) {
        prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v); prefetch_tensormap(&tm_o);
    }
    __syncthreads();
    if (warp == 9) tmem_alloc_2sm(smem_u32(&tmem_slot), TMEM_COLS);
    tc_fence_before();
    cluster_sync_all();                                   // both CTAs' barriers and TMEM exist before anyone uses them
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const int G = gridDim.x >> 1;
    const int n_rounds = (n_items + G - 1) / G;
    // the leader's barriers that the peer signals
    const uint32_t lead_ofree = map_to_cta(smem_u32(&bar_ofree), 0);
    uint32_t lead_pf[kNU];
#pragma unroll
    for (int i = 0; i < kNU; i++) lead_pf[i] = map_to_cta(smem_u32(&bar_pf[i]), 0);

    if (warp >= 8) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));

    if (warp == 8) {
        // ------------------------------------------------------------ TMA producer: Q and the K halves
        if (lane == 0) {
            int g = 0, it_n = 0, g_item0 = 0;
            bool ok = true;
            for (int r = 0; ok && r < n_rounds; r++) {
                Item2 it;
                if (!get_item2<CAUSAL>(r, n_items, n_bh, n_pairs, seq_len, heads_per_group, it)) continue;
                // Q is free after the previous item's last Q K^T (entry of that tile in the ring)
                if (it_n > 0 && !mbar_wait(smem_u32(&bar_qk[(g_item0 - 1) % kRing]), ((g_item0 - 1) / kRing) & 1, ctl, k2QFree)) break;
                if (leader) mbar_arrive_expect_tx(smem_u32(&bar_qf), 2 * L::kQBytes);    // both CTAs' query tiles
                for (int b = 0; b < NBOX; b++)
                    tma_load_3d_2sm(q_s + b * L::kBox, &tm_q, smem_u32(&bar_qf), b * 64,
                                    (2 * it.pair + static_cast<int>(rank)) * kBM, it.bh);
                for (int j = 0; j < it.n_kv; j++, g++) {
                    const int sk = g % kStages;
                    // the slot was last read by Q K^T of tile g - kStages
                    if (g >= kStages && !mbar_wait(smem_u32(&bar_qk[(g - kStages) % kRing]), ((g - kStages) / kRing) & 1, ctl, k2KFree)) { ok = false; break; }
                    if (leader) mbar_arrive_expect_tx(smem_u32(&bar_kf[sk]), 2 * L::kKHalf);
                    for (int b = 0; b < NBOX; b++)       // this CTA's 64 keys of the tile
                        tma_load_3d_2sm(k_s + sk * L::kKHalf + b * (64 * 128), &tm_k, smem_u32(&bar_kf[sk]), b * 64,
                                        j * kBN + static_cast<int>(rank) * 64, it.bh);
                }
                it_n++;
                g_item0 = g;
            }
        }
        __syncwarp();
    } else if (warp == 11) {
        // ------------------------------------------------------------ TMA producer: the V halves
        if (lane == 0) {
            int g = 0;
            bool ok = true;
            for (int r = 0; ok && r < n_rounds; r++) {
                Item2 it;
                if (!get_item2<CAUSAL>(r, n_items, n_bh, n_pairs, seq_len, heads_per_group, it)) continue;
                for (int j = 0; j < it.n_kv; j++, g++) {
                    const int sv = g % kStages;
                    if (g >= kStages && !mbar_wait(smem_u32(&bar_pvd[(g - kStages) % kRing]), ((g - kStages) / kRing) & 1, ctl, k2VFree)) { ok = false; break; }
                    if (leader) mbar_arrive_expect_tx(smem_u32(&bar_vf[sv]), 2 * L::kVHalf);
                    // this CTA's 64 head-dim columns of the tile's 128 keys
                    tma_load_3d_2sm(v_s + sv * L::kVHalf, &tm_v, smem_u32(&bar_vf[sv]), static_cast<int>(rank) * 64,
                                    j * kBN, it.bh);
                }
            }
        }
        __syncwarp();
    } else if (warp == 9) {
        // ------------------------------------------------------------ Q K^T issuer (leader CTA only)
        if (leader && lane == 0) {
            constexpr uint32_t idesc_qk = make_idesc(2 * kBM, kBN, FMT, FMT, kMajorK, kMajorK);
            constexpr uint64_t hi_k = make_sdesc_hi(16, 1024);
            int g = 0, it_n = 0, u = 0;
            bool ok = true;
            for (int r = 0; ok && r < n_rounds; r++) {
                Item2 it;
                if (!get_item2<CAUSAL>(r, n_items, n_bh, n_pairs, seq_len, heads_per_group, it)) continue;
                if (!mbar_wait_cluster(smem_u32(&bar_qf), it_n & 1, ctl, k2QFull)) break;
                for (int j = 0; j < it.n_kv; j++, g++) {
                    const int sk = g % kStages;
                    if (!mbar_wait_cluster(smem_u32(&bar_kf[sk]), (g / kStages) & 1, ctl, k2KFull)) { ok = false; break; }
                    // the score buffer last held S and then P of tile g - kNU: that P V must be done
                    if (g >= kNU && !mbar_wait(smem_u32(&bar_pvd[(g - kNU) % kRing]), ((g - kNU) / kRing) & 1, ctl, k2SFree)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t kb = k_s + sk * L::kKHalf;
                    const uint32_t sc = tmem + u * 128;
#pragma unroll
                    for (int kk = 0; kk < D / 16; kk++) {
                        const uint32_t qoff = (kk >> 2) * L::kBox + (kk & 3) * 32;
                        const uint32_t koff = (kk >> 2) * (64 * 128) + (kk & 3) * 32;
                        mma_f16_ss_2sm(sc, make_sdesc(q_s + qoff, hi_k), make_sdesc(kb + koff, hi_k), idesc_qk, kk > 0);
                    }
                    tc_commit_2sm(smem_u32(&bar_qk[g % kRing]));      // both CTAs: S ready, K slot free, (last tile) Q free
                    u = (u == kNU - 1) ? 0 : u + 1;
                }
                it_n++;
            }
        }
        __syncwarp();
    } else if (warp == 10) {
        // ------------------------------------------------------------ P V issuer (leader CTA only)
        if (leader && lane == 0) {
            constexpr uint32_t idesc_pv = make_idesc(2 * kBM, D, FMT, FMT, kMajorK, kMajorMN);
            constexpr uint64_t hi_v = make_sdesc_hi(L::kBox, 1024);
            int g = 0, it_n = 0, u = 0, u_phase = 0;
            bool ok = true;
            for (int r = 0; ok && r < n_rounds; r++) {
                Item2 it;
                if (!get_item2<CAUSAL>(r, n_items, n_bh, n_pairs, seq_len, heads_per_group, it)) continue;
                for (int j = 0; j < it.n_kv; j++, g++) {
                    const int sv = g % kStages;
                    if (!mbar_wait_cluster(smem_u32(&bar_vf[sv]), (g / kStages) & 1, ctl, k2VFull)) { ok = false; break; }
                    if (!mbar_wait_cluster(smem_u32(&bar_pf[u]), u_phase, ctl, k2PFull)) { ok = false; break; }
                    // the first P V of an item overwrites O: both CTAs' epilogues must have read the previous one
                    if (j == 0 && it_n > 0 && !mbar_wait_cluster(smem_u32(&bar_ofree), (it_n - 1) & 1, ctl, k2OFree)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t vb = v_s + sv * L::kVHalf;
                    const uint32_t pc = tmem + u * 128;
#pragma unroll
                    for (int kk = 0; kk < kBN / 16; kk++)
                        mma_f16_ts_2sm(tmem + O_COL, pc + kk * 8, make_sdesc(vb + kk * 2048, hi_v), idesc_pv,
                                       (j > 0 || kk > 0) ? 1u : 0u);
                    tc_commit_2sm(smem_u32(&bar_pvd[g % kRing]));     // both CTAs: score buffer and V slot free, (last tile) O done
                    if (u == kNU - 1) { u = 0; u_phase ^= 1; } else { u++; }
                }
                it_n++;
            }
        }
        __syncwarp();
    } else if (warp >= 12) {
        // ------------------------------------------------------------ epilogue warps 12-15 (each CTA: its own tile)
        const int r_in_tile = tid - 384;
        const uint32_t t_o = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + O_COL;
        int n_rv = 0;
        auto rendezvous4 = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_epi));
            const bool w = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_epi), n_rv & 1, ctl, k2Epi));
            n_rv++;
            return w;
        };
        int it_n = 0, g = 0;
        for (int r = 0; r < n_rounds; r++) {
            Item2 it;
            if (!get_item2<CAUSAL>(r, n_items, n_bh, n_pairs, seq_len, heads_per_group, it)) continue;
            g += it.n_kv;
            const int q_start = (2 * it.pair + static_cast<int>(rank)) * kBM;
            const int par = it_n & 1;
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_stats[par]), (it_n >> 1) & 1, ctl, k2Stats))) break;
            const float m_a = xm[par][0][r_in_tile], m_b = xm[par][1][r_in_tile];
            const float m_fin = fmaxf(m_a, m_b);
            const float l_run = xsum[par][0][r_in_tile] * ex2_approx(m_a - m_fin) +
                                xsum[par][1][r_in_tile] * ex2_approx(m_b - m_fin);
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_stats_free[par]));
            const float inv_l = 1.0f / l_run;
            const int row = q_start + r_in_tile;
            if (lse_out != nullptr && row < seq_len)
                lse_out[static_cast<size_t>(it.bh) * seq_len + row] = kLn2 * (m_fin + log2f(l_run));
            // O is complete when the item's last P V is
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_pvd[(g - 1) % kRing]), ((g - 1) / kRing) & 1, ctl, k2ODone))) break;
            tc_fence_after();
            if (tid == 384) tma_store_wait_read();        // staging drained by the previous item's store
            if (!rendezvous4()) break;
#pragma unroll 1
            for (int c = 0; c < D / 32; c++) {
                uint32_t o[32];
                tmem_ld32_wait(t_o + c * 32, o);
                if (c == D / 32 - 1) {                    // the row is out of TMEM: tell the leader's P V issuer
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_remote(lead_ofree);
                }
#pragma unroll
                for (int g8 = 0; g8 < 4; g8++) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; e++)
                        w[e] = pack_16<BF16>(__uint_as_float(o[g8 * 8 + 2 * e]) * inv_l,
                                             __uint_as_float(o[g8 * 8 + 2 * e + 1]) * inv_l);
                    const int c16 = c * 4 + g8;
                    const uint32_t addr = o_s + (c16 >> 3) * L::kBox + r_in_tile * 128 +
                                          (((c16 & 7) ^ (r_in_tile & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]),
                                 "r"(w[2]), "r"(w[3]) : "memory");
                }
            }
            fence_proxy_async_smem();
            if (!rendezvous4()) break;
            if (tid == 384 && q_start < seq_len) {        // the odd tile of the last pair may lie past the sequence
                for (int bx = 0; bx < NBOX; bx++)
                    tma_store_3d(&tm_o, o_s + bx * L::kBox, bx * 64, q_start, it.bh);
                tma_store_commit();
            }
            it_n++;
        }
        if (tid == 384) tma_store_wait_read();
        __syncwarp();
    } else {
        // ------------------------------------------------------------ softmax (warps 0-7), each CTA on its own tile
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
        const int grp = warp >> 2;                        // group 0 owns even key tiles, group 1 odd ones
        const int r_in_tile = (warp & 3) * 32 + lane;
        const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t t_o = tmem + lane_off + O_COL;
        const uint64_t scale2 = pack2(scale_log2, scale_log2);
        int g0 = 0, it_n = 0;
        bool ok = true;

        for (int r = 0; ok && r < n_rounds; r++) {
            Item2 it;
            if (!get_item2<CAUSAL>(r, n_items, n_bh, n_pairs, seq_len, heads_per_group, it)) continue;
            const int q_start = (2 * it.pair + static_cast<int>(rank)) * kBM;
            const int row = q_start + r_in_tile;
            const int row_limit = CAUSAL ? min(seq_len, row + 1) : seq_len;
            const int tile_min_limit = CAUSAL ? min(seq_len, q_start + 1) : seq_len;
            float m_mine = -1e30f;
            uint64_t lsum2 = pack2(0.0f, 0.0f);

            for (int j = (g0 & 1) == grp ? 0 : 1; j < it.n_kv; j += 2) {
                const int g = g0 + j;
                const int kv_start = j * kBN;
                if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_qk[g % kRing]), (g / kRing) & 1, ctl, k2SFull))) { ok = false; break; }
                tc_fence_after();
                const int u = g % kNU;
                const uint32_t t_s = tmem + lane_off + u * 128;
                uint32_t s[128];
                tmem_ld128_wait(t_s, s);
                if ((tile_min_limit - kv_start) < kBN) {  // tile touches the mask or the ragged end (or lies wholly behind it)
                    const int limit = row_limit - kv_start;
#pragma unroll
                    for (int i = 0; i < 128; i++) s[i] = (i < limit) ? s[i] : 0xff800000u;
                }
                float a0 = -INFINITY, a1 = -INFINITY, a2 = -INFINITY, a3 = -INFINITY;
#pragma unroll
                for (int i = 0; i < 128; i += 8) {
                    a0 = max3(a0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
                    a1 = max3(a1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
                    a2 = max3(a2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
                    a3 = max3(a3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
                }
                const float tile_max = fmaxf(max3(a0, a1, a2), a3) * scale_log2;
                float m_new = tile_max, m_prev_keep = tile_max;
                bool changed = false;
                const uint32_t slot = smem_u32(&m_slot[it_n & 1][r_in_tile]);
                if (j > 0) {
                    uint32_t mb = 0, tag = 0;
                    const int w = bounded_wait(
                        [&] {
                            asm volatile("ld.volatile.shared.v2.b32 {%0, %1}, [%2];" : "=r"(mb), "=r"(tag) : "r"(slot));
                            return tag == static_cast<uint32_t>(g - 1);
                        },
                        [&] { return *ctl.abort_flag != 0; }, [] { return global_timer_ns(); }, kWaitLimitNs, 256u);
                    if (!__all_sync(0xffffffffu, w == kWaitDone)) {
                        if (w == kWaitTimedOut) {
                            *ctl.abort_flag = 1;
                            atomicCAS(ctl.status, 0, wait_timeout_word(k2M));
                        }
                        ok = false;
                        break;
                    }
                    const float m_prev = __uint_as_float(mb);
                    m_prev_keep = m_prev;
                    changed = tile_max > m_prev + kRescaleThreshold;
                    m_new = changed ? tile_max : m_prev;
                }
                asm volatile("st.volatile.shared.v2.b32 [%0], {%1, %2};" ::"r"(slot), "r"(__float_as_uint(m_new)),
                             "r"(static_cast<uint32_t>(g)) : "memory");
                if (m_new != m_mine) {
                    const float f = ex2_approx(m_mine - m_new);
                    lsum2 = fma2(lsum2, pack2(f, f), pack2(0.0f, 0.0f));
                }
                if (__any_sync(0xffffffffu, changed)) {
                    // P V(g-1) must have finished accumulating into O
                    if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_pvd[(g - 1) % kRing]), ((g - 1) / kRing) & 1, ctl, k2PV))) { ok = false; break; }
                    tc_fence_after();
                    const float factor = changed ? ex2_approx(m_prev_keep - m_new) : 1.0f;
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
                m_mine = m_new;

                const uint64_t negm2 = pack2(-m_new, -m_new);
                uint64_t acc0 = lsum2, acc1 = pack2(0.0f, 0.0f), acc2 = acc1, acc3 = acc1;
                constexpr int NCHUNK = 4;
                constexpr int PAIRS = 64 / NCHUNK;
#pragma unroll
                for (int c = 0; c < NCHUNK; c++) {
                    uint32_t pk[PAIRS];
#pragma unroll
                    for (int i = 0; i < PAIRS; i++) {
                        const int e = 2 * (c * PAIRS + i);
                        const uint64_t x = fma2(pack2(__uint_as_float(s[e]), __uint_as_float(s[e + 1])), scale2, negm2);
                        float x0, x1;
                        unpack2(x, x0, x1);
                        const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
                        const uint64_t pp = pack2(p0, p1);
                        if ((i & 3) == 0) acc0 = add2(acc0, pp);
                        else if ((i & 3) == 1) acc1 = add2(acc1, pp);
                        else if ((i & 3) == 2) acc2 = add2(acc2, pp);
                        else acc3 = add2(acc3, pp);
                        pk[i] = pack_16<BF16>(p0, p1);
                    }
                    tmem_st_x16(t_s + c * PAIRS, pk);
                }
                lsum2 = add2(add2(acc0, acc1), add2(acc2, acc3));
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(lead_pf[u]);       // the leader's P V issuer waits for both CTAs
            }
            if (!ok) break;
            {
                const int par = it_n & 1;
                if (it_n >= 2 &&
                    !__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_stats_free[par]), ((it_n >> 1) - 1) & 1, ctl, k2StatsFree))) { ok = false; break; }
                float l0, l1;
                unpack2(lsum2, l0, l1);
                xm[par][grp][r_in_tile] = m_mine;
                xsum[par][grp][r_in_tile] = l0 + l1;
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar_stats[par]));
            }
            g0 += it.n_kv;
            it_n++;
        }
    }

    // No CTA may leave while its peer can still signal its barriers, read its shared memory through
    // an MMA or write its TMEM.
    tc_fence_before();
    cluster_sync_all();
    if (warp == 9) tmem_dealloc_2sm(tmem, TMEM_COLS);
}

template <int D, bool CAUSAL, bool BF16>
int launch_2sm_instance(const fa_prefill_args& a, DeviceState* st, int heads_per_group, const CUtensorMap& tq,
                        const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to) {
    using L = PairSmem2<D>;
    auto kernel = prefill_2sm_kernel<D, CAUSAL, BF16>;
    static bool configured[64] = {};
    if (!configured[st->device]) {
        FA_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
        configured[st->device] = true;
    }
    const int n_bh = a.batch_size * a.num_heads;
    const int n_qtiles = (a.seq_len + kBM - 1) / kBM;
    const int n_pairs = (n_qtiles + 1) / 2;
    const long long n_items = (long long)n_bh * n_pairs;
    if (n_items > 0x7FFFFFFFll) return FA_ERR_INVALID_ARGUMENT;
    const int max_clusters = st->sm_count / 2;
    const unsigned clusters = (unsigned)(n_items < max_clusters ? n_items : max_clusters);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * clusters);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = L::kTotal;
    cfg.stream = static_cast<cudaStream_t>(a.stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    FA_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, tq, tk, tv, to, a.lse, a.seq_len, n_bh, n_pairs, (int)n_items,
                                   heads_per_group, a.scale * kLog2e, st->status));
    return FA_OK;
}

}  // namespace

// d_head 128, fp16 / bf16.  The K tensor map has boxes of 64 keys, the V map boxes of 128 keys x 64 columns.
int launch_prefill_2sm_16bit(const fa_prefill_args& a, DeviceState* st, int heads_per_group) {
    const uint64_t n_bh = (uint64_t)a.batch_size * a.num_heads;
    CUtensorMap tq, tk, tv, to;
    int rc;
    if ((rc = make_tensor_map_3d(&tq, a.q, a.dtype, a.d_head, a.seq_len, n_bh, 64, kBM)) != FA_OK) return rc;
    if ((rc = make_tensor_map_3d(&tk, a.k, a.dtype, a.d_head, a.seq_len, n_bh, 64, 64)) != FA_OK) return rc;
    if ((rc = make_tensor_map_3d(&tv, a.v, a.dtype, a.d_head, a.seq_len, n_bh, 64, kBN)) != FA_OK) return rc;
    if ((rc = make_tensor_map_3d(&to, a.o, a.dtype, a.d_head, a.seq_len, n_bh, 64, kBM)) != FA_OK) return rc;
    const bool bf = a.dtype == FA_DTYPE_BF16;
    if (a.causal) return bf ? launch_2sm_instance<128, true, true>(a, st, heads_per_group, tq, tk, tv, to)
                            : launch_2sm_instance<128, true, false>(a, st, heads_per_group, tq, tk, tv, to);
    return bf ? launch_2sm_instance<128, false, true>(a, st, heads_per_group, tq, tk, tv, to)
              : launch_2sm_instance<128, false, false>(a, st, heads_per_group, tq, tk, tv, to);
}

}  // namespace fa
