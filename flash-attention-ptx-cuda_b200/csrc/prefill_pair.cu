// Prefill forward kernel for sm_100a with TWO query tiles in flight per CTA:
// fp16 / bf16, d_head 64 or 128, causal or not, any sequence length.
//
// Replaces the reference's kernel and launcher for problems large enough to fill
// the GPU (kernels/flash_attention.cu:116-507 flash_attention_ptx_kernel, :534-579
// launch_variant; the reference's own dispatcher, :595-617, likewise picks a tile
// variant by problem size).  Same mathematics as the reference - per query row an
// online softmax over key tiles with a running max and sum (:332-401), O += P V
// (:437-468), rescale when the max moves (:411-425), O / sum and
// LSE = max + log(sum) at the end (:476-505) - none of its structure.
//
// A work item is a pair of adjacent 128-row query tiles (A, B) of one (batch, head).
// Every K / V tile in shared memory feeds both tiles: two Q K^T and two P V products
// per tile loaded, and the two tiles' chains  Q K^T -> softmax -> P V  are independent,
// so while one tile's scores are exponentiated the tensor pipe works for the other.
//
//   warps 0-3 / 4-7   softmax of tile A / tile B.  A thread owns a query row (TMEM lane):
//                     one tcgen05.ld brings the 128 scores of a key tile into registers,
//                     the running max and sum live in registers, p = 2^(s*scale*log2e - m)
//                     goes back to TMEM as 16-bit pairs.  The max in use only moves (and O
//                     is only rescaled, in TMEM, by the row's thread) when a tile's max
//                     exceeds it by more than 2^8.
//   warp 8            TMA producer: Q of both tiles per item, the K ring.
//   warp 11           TMA producer: the V ring (a V slot frees much later than a K slot).
//   warp 9 / warp 10  MMA issuer of tile A / tile B (lane 0 issues): S = Q K^T into the
//                     tile's score buffer, O += P V with P from TMEM and V (MN-major) from
//                     shared memory.  Instructions of one thread execute in order, which is
//                     what lets P alias S at d_head 128.
//   warps 12-15       epilogue, one thread per row: O / l -> 16-bit -> swizzled staging ->
//                     TMA store (clipped per head), tile A then tile B, while the other
//                     roles are already on the next item.
//
// TMEM (512 columns):
//   d_head 64 :  S_A [0,128) S_B [128,256) P_A [256,320) P_B [320,384) O_A [384,448) O_B [448,512)
//                P has its own columns, so Q K^T of the next key tile is issued as soon as
//                the softmax has READ the scores: a softmax group goes from tile to tile
//                without waiting for the tensor pipe (at d_head 64 the exponentials, not the
//                tensor pipe, are the longer half).
//   d_head 128:  S_A [0,128) S_B [128,256) O_A [256,384) O_B [384,512); P overwrites the
//                first 64 columns of the scores it came from.
//
// Every wait is bounded; on expiry the CTA records (1 << 16) | barrier id in the device
// status word and every role leaves its loops.
#include <cmath>
#include <type_traits>

#include "host_common.h"
#include "ptx.cuh"
#include "tmem_ld.cuh"

// Cycle-accounting hooks: no-ops unless a development build defines them before this point.
#ifndef FA_PROBE_DECL
#define FA_PROBE_DECL
#define FA_PROBE(k) do {} while (0)
#define FA_PROBE_FLUSH(role, count) do {} while (0)
#endif

namespace fa {
namespace {

constexpr int kBM = 128;                 // query rows per tile (two tiles per work item)
constexpr int kBN = 128;                 // keys per tile
constexpr int kThreads = 512;
// setmaxnreg moves registers inside the pool the CTA got at launch (threads x registers at launch).
constexpr int kRegsLaunch = (65536 / kThreads) / 8 * 8;
constexpr int kRegsSoftmax = 192;        // warps 0-7
constexpr int kRegsOther = 64;           // warps 8-15
static_assert(256 * kRegsSoftmax + 256 * kRegsOther <= kThreads * kRegsLaunch,
              "setmaxnreg targets exceed the CTA's register pool");
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;   // log2 units: rescale only if the max grew by more than 2^8
// The exponentials are the longest pole at d_head 64 (16 per clock per SM on the special-function
// unit: 1024 clocks per 128 x 128 score tile, against 512 clocks of tensor work), so every
// kPolyEvery-th pair of scores is exponentiated on the FMA pipe instead (0 = none).
constexpr int kPolyEvery = 0;

// 2^x for two values on the FMA pipe: x = n + f with n = round(x), f in [-1/2, 1/2];
// 2^f by a cubic (max relative error 7.5e-5, below the rounding of P to 16 bits), times 2^n by
// adding n to the exponent field.  x is clamped to >= -120 so that the exponent stays in range
// (masked scores, -inf, come out as 2^-120, i.e. zero for every purpose here); callers keep
// x <= 8 + a few.
__device__ __forceinline__ void exp2_pair_fma(uint64_t x2, float& p0, float& p1) {
    float x0, x1;
    unpack2(x2, x0, x1);
    x2 = pack2(fmaxf(x0, -120.0f), fmaxf(x1, -120.0f));
    constexpr float kMagic = 12582912.0f;           // 1.5 * 2^23: adding it leaves round(x) in the low mantissa bits
    const uint64_t t2 = add2(x2, pack2(kMagic, kMagic));
    const uint64_t n2 = add2(t2, pack2(-kMagic, -kMagic));
    const uint64_t f2 = fma2(n2, pack2(-1.0f, -1.0f), x2);
    uint64_t q2 = fma2(f2, pack2(0.05517144873738289f, 0.05517144873738289f), pack2(0.2426108419895172f, 0.2426108419895172f));
    q2 = fma2(q2, f2, pack2(0.6932609677314758f, 0.6932609677314758f));
    q2 = fma2(q2, f2, pack2(0.9999281167984009f, 0.9999281167984009f));
    float t0, t1, q0, q1;
    unpack2(t2, t0, t1);
    unpack2(q2, q0, q1);
    p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(t0) << 23));
    p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(t1) << 23));
}

// Barrier ids reported in the status word when a wait gives up (0x40 + ...: this kernel).
enum : int { kPQFull = 0x41, kPQFree, kPKFull, kPKFree, kPVFull, kPVFree, kPSFull, kPSFree, kPPFull,
             kPPvDone, kPODone, kPOFree, kPStatsFull, kPStatsFree, kPEpi };

constexpr int kMaxStages = 4;
constexpr int kRing = 8;                 // entries of the completion rings; must exceed the K / V stage counts

// Control block at the start of dynamic shared memory: every mbarrier of the kernel and the
// softmax -> epilogue hand-off of 1 / row sum.
//
// A tcgen05.commit stalls its thread for ~200 clocks while MMAs are in flight (measured), so an
// issuer commits exactly ONCE per product, onto a ring entry chosen by the query tile's running
// key-tile count t (entry t % kRing, phase (t / kRing) & 1), and every role that cares about that
// product waits on the same entry:
//   s_full[X][.]   Q K^T of chain tile t is done: the softmax may read S; the K slot is free once
//                  both query tiles' entries for that key tile are complete; Q is free after the
//                  item's last one.
//   pv_done[X][.]  P V of chain tile t is done: the V slot is free (both tiles' entries); P's columns
//                  may change (d_head 64); after the item's last one O is complete.
// A ring entry is reused kRing tiles later; no waiter can fall that far behind, because the tile
// that reuses the entry needs a K / V slot, a P or an O that the waiter itself hands over.
struct PairCtrl {
    uint64_t q_full[2];                               // per query tile: Q landed
    uint64_t k_full[kMaxStages], v_full[kMaxStages];  // K / V tile landed
    uint64_t s_full[2][kRing], pv_done[2][kRing];     // completion rings of the two products, per query tile
    uint64_t s_free[2];                               // scores read into registers (d_head 64: S may be overwritten)
    uint64_t p_full[2];                               // P of a key tile is in TMEM
    uint64_t o_free[2];                               // the epilogue has read O
    uint64_t stats_full[2], stats_free[2];
    uint64_t epi;                                     // rendezvous of the four epilogue warps
    float    inv_l[2][128];
    uint32_t tmem_slot;
    int      abort_flag;
};

template <int D>
struct PairSmem {
    static constexpr int kNBox  = D / 64;               // 64-column (128-byte) boxes per 16-bit row
    static constexpr int kBox   = 128 * 128;            // one box: 128 rows x 128 bytes
    static constexpr int kTile  = kNBox * kBox;         // one 128 x D 16-bit tile
    static constexpr int NK     = (D == 64) ? 4 : 2;
    static constexpr int NV     = (D == 64) ? 4 : 2;
    static constexpr int NO     = (D == 64) ? 2 : 1;    // output staging tiles
    static constexpr int kCtrl  = (sizeof(PairCtrl) + 127) / 128 * 128;
    static constexpr int kTotal = kCtrl + 1024 + (2 + NK + NV + NO) * kTile;
    static_assert(NK <= kMaxStages && NV <= kMaxStages && kMaxStages < kRing, "ring size");
    static_assert(kTotal <= 232448, "shared memory per CTA");
};

// Work list: pairs of query tiles, heaviest first under the causal mask, dealt to the CTAs in
// boustrophedon order so that the per-CTA totals even out.
struct PairItem {
    int bh;
    int qa;        // first query row of tile A; tile B starts at qa + 128
    int n_a, n_b;  // key tiles tile A / tile B walks (n_b == 0: the sequence ends inside tile A)
    int n;         // key tiles loaded for the item = max(n_a, n_b)
};

template <bool CAUSAL>
__device__ __forceinline__ bool get_pair_item(int round, int n_items, int n_bh, int n_pairs, int seq_len,
                                              int heads_per_group, PairItem& it) {
    const int G = gridDim.x, c = blockIdx.x;
    const int idx = (round & 1) ? round * G + (G - 1 - c) : round * G + c;
    if (idx >= n_items) return false;
    // Heads are walked in groups whose K/V fit in L2 together (one group = all heads when the
    // whole problem fits); inside a group the order is (pair, head) as before.
    const int per_group = heads_per_group * n_pairs;
    const int gi = idx / per_group, rem = idx - gi * per_group;
    const int h0 = gi * heads_per_group, hin = min(heads_per_group, n_bh - h0);
    const int rank = rem / hin;
    const int pr = CAUSAL ? (n_pairs - 1 - rank) : rank;
    it.bh = h0 + rem - rank * hin;
    it.qa = pr * 2 * kBM;
    const int n_all = (seq_len + kBN - 1) / kBN;
    const bool has_b = it.qa + kBM < seq_len;
    it.n_a = CAUSAL ? min(n_all, 2 * pr + 1) : n_all;
    it.n_b = has_b ? (CAUSAL ? min(n_all, 2 * pr + 2) : n_all) : 0;
    it.n = max(it.n_a, it.n_b);
    return true;
}

template <int D, bool CAUSAL, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
prefill_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                    float* __restrict__ lse_out, int seq_len, int n_bh, int n_pairs, int n_items,
                    int heads_per_group, float scale_log2, int* status) {
    using L = PairSmem<D>;
    constexpr int NBOX = L::kNBox, NK = L::NK, NV = L::NV, NO = L::NO;
    constexpr bool INPLACE = (D == 128);                  // P overwrites the scores it came from
    constexpr uint32_t S_COL0 = 0, S_COL1 = 128;
    constexpr uint32_t P_COL0 = INPLACE ? S_COL0 : 256, P_COL1 = INPLACE ? S_COL1 : 320;
    constexpr uint32_t O_COL0 = INPLACE ? 256 : 384, O_COL1 = INPLACE ? 384 : 448;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t FMT = BF16 ? kFmtBF16 : kFmtF16;

    extern __shared__ uint8_t smem_raw[];
    PairCtrl& cb = *reinterpret_cast<PairCtrl*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t base = (smem_u32(smem_raw) + L::kCtrl + 1023u) & ~1023u;
    const uint32_t q_s = base;                            // Q_A, Q_B
    const uint32_t k_s = q_s + 2 * L::kTile;
    const uint32_t v_s = k_s + NK * L::kTile;
    const uint32_t o_s = v_s + NV * L::kTile;
    WaitCtl ctl{&cb.abort_flag, status};

    if (tid == 0) {
        for (int x = 0; x < 2; x++) {
            mbar_init(smem_u32(&cb.q_full[x]), 1);
            for (int i = 0; i < kRing; i++) {
                mbar_init(smem_u32(&cb.s_full[x][i]), 1);
                mbar_init(smem_u32(&cb.pv_done[x][i]), 1);
            }
            mbar_init(smem_u32(&cb.s_free[x]), 4);        // one arrival per warp of the tile's softmax group
            mbar_init(smem_u32(&cb.p_full[x]), 4);
            mbar_init(smem_u32(&cb.o_free[x]), 4);        // the epilogue warps have read O
            mbar_init(smem_u32(&cb.stats_full[x]), 4);
            mbar_init(smem_u32(&cb.stats_free[x]), 4);
        }
        for (int i = 0; i < kMaxStages; i++) {
            mbar_init(smem_u32(&cb.k_full[i]), 1);
            mbar_init(smem_u32(&cb.v_full[i]), 1);
        }
        mbar_init(smem_u32(&cb.epi), 4);
        cb.abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 8 && lane == 0) {
        prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v); prefetch_tensormap(&tm_o);
    }
    __syncthreads();
    if (warp == 9) tmem_alloc(smem_u32(&cb.tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = cb.tmem_slot;
    const int n_rounds = (n_items + gridDim.x - 1) / gridDim.x;
    // waits until product `t` of query tile X has completed (t < 0: nothing to wait for)
    auto wait_qk_done = [&](int X, int t, int id) -> bool {
        return t < 0 || mbar_wait(smem_u32(&cb.s_full[X][t % kRing]), (t / kRing) & 1, ctl, id);
    };
    auto wait_pv_done = [&](int X, int t, int id) -> bool {
        return t < 0 || mbar_wait(smem_u32(&cb.pv_done[X][t % kRing]), (t / kRing) & 1, ctl, id);
    };

    if (warp >= 8) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));

    // Roles of warps 8-11: K (and Q) producer, one MMA issuer per query tile, V producer.  One thread
    // issues both products of its query tile: at d_head 128, where P aliases S, that is what orders
    // P V(j) before Q K^T(j + 1); at d_head 64 it keeps the two query tiles' chains independent of
    // each other (a shared Q K^T issuer made tile A wait whenever tile B was behind).
    constexpr int kWarpLoadKV = 8, kWarpLoadV = 11;
    constexpr int kWarpChainA = 9, kWarpChainB = 10;

    if (warp == kWarpLoadKV || warp == kWarpLoadV) {
        // ------------------------------------------------------------ TMA producer(s)
        const bool do_k = warp == kWarpLoadKV;            // Q and K
        const bool do_v = warp == kWarpLoadV;
        if (lane == 0) {
            int g = 0, it_a = 0, it_b = 0;                // K/V tiles loaded; items seen with a tile A / B
            int t_a = 0, t_b = 0;                         // key tiles of query tile A / B before this item
            // per ring slot: the chain tiles (A's and B's count, -1 = none) whose product last read it
            int k_user[2][kMaxStages], v_user[2][kMaxStages];
            bool ok = true;
            for (int r = 0; ok && r < n_rounds; r++) {
                PairItem it;
                if (!get_pair_item<CAUSAL>(r, n_items, n_bh, n_pairs, seq_len, heads_per_group, it)) continue;
                for (int j = 0; j < it.n; j++, g++) {
                    const int ua = j < it.n_a ? t_a + j : -1, ub = j < it.n_b ? t_b + j : -1;
                    if (do_k) {
                        if (j == 0) {
                            // Q_A goes first: with K(0) it is all the item's first Q K^T needs.  The
                            // buffer is free after the previous item's last Q K^T of this query tile.
                            if (!wait_qk_done(0, t_a - 1, kPQFree)) { ok = false; break; }
                            mbar_arrive_expect_tx(smem_u32(&cb.q_full[0]), L::kTile);
                            for (int b = 0; b < NBOX; b++)
                                tma_load_3d(q_s + b * L::kBox, &tm_q, smem_u32(&cb.q_full[0]), b * 64, it.qa, it.bh);
                            it_a++;
                        }
                        const int sk = g % NK;
                        if (g >= NK && !(wait_qk_done(0, k_user[0][sk], kPKFree) && wait_qk_done(1, k_user[1][sk], kPKFree))) { ok = false; break; }
                        k_user[0][sk] = ua; k_user[1][sk] = ub;
                        mbar_arrive_expect_tx(smem_u32(&cb.k_full[sk]), L::kTile);
                        for (int b = 0; b < NBOX; b++)
                            tma_load_3d(k_s + sk * L::kTile + b * L::kBox, &tm_k, smem_u32(&cb.k_full[sk]), b * 64,
                                        j * kBN, it.bh);
                        if (j == 0 && it.n_b > 0) {
                            if (!wait_qk_done(1, t_b - 1, kPQFree)) { ok = false; break; }
                            mbar_arrive_expect_tx(smem_u32(&cb.q_full[1]), L::kTile);
                            for (int b = 0; b < NBOX; b++)
                                tma_load_3d(q_s + L::kTile + b * L::kBox, &tm_q, smem_u32(&cb.q_full[1]), b * 64,
                                            it.qa + kBM, it.bh);
                            it_b++;
                        }
                    }
                    if (do_v) {
                        const int sv = g % NV;
                        if (g >= NV && !(wait_pv_done(0, v_user[0][sv], kPVFree) && wait_pv_done(1, v_user[1][sv], kPVFree))) { ok = false; break; }
                        v_user[0][sv] = ua; v_user[1][sv] = ub;
                        mbar_arrive_expect_tx(smem_u32(&cb.v_full[sv]), L::kTile);
                        for (int b = 0; b < NBOX; b++)
                            tma_load_3d(v_s + sv * L::kTile + b * L::kBox, &tm_v, smem_u32(&cb.v_full[sv]), b * 64,
                                        j * kBN, it.bh);
                    }
                }
                t_a += it.n_a; t_b += it.n_b;
            }
        }
        __syncwarp();
    } else if (warp == kWarpChainA || warp == kWarpChainB) {
        // ------------------------------------------------------------ MMA issuers
        // One thread (lane 0) runs its whole loop.  (Measured in isolation: one thread issuing back
        // to back needs ~55-63 clocks per tcgen05.mma, a warp-uniform loop with a predicated issue
        // per instruction ~70-76; next to busy softmax warps about 100.)
        if (lane == 0) {
        constexpr uint32_t idesc_qk = make_idesc(kBM, kBN, FMT, FMT, kMajorK, kMajorK);
        constexpr uint32_t idesc_pv = make_idesc(kBM, D, FMT, FMT, kMajorK, kMajorMN);
        constexpr uint64_t hi_k = make_sdesc_hi(16, 1024);
        constexpr uint64_t hi_v = make_sdesc_hi(L::kBox, 1024);
        int t[2] = {0, 0}, itx[2] = {0, 0};               // per query tile: key tiles / items so far
        int g0 = 0;                                       // K/V tiles of all items so far
        FA_PROBE_DECL

        // S = Q K^T of query tile X against the item's key tile j (tile t[X] + j of that chain).
        auto issue_qk = [&](int X, int j) -> bool {
            const int gk = g0 + j, sk = gk % NK;
            if (!mbar_wait(smem_u32(&cb.k_full[sk]), (gk / NK) & 1, ctl, kPKFull)) return false;
            FA_PROBE(0);
            if constexpr (!INPLACE) {
                // the softmax must have read the previous scores out of the buffer
                if (t[X] + j > 0 && !mbar_wait(smem_u32(&cb.s_free[X]), (t[X] + j - 1) & 1, ctl, kPSFree)) return false;
            }
            tc_fence_after();
            FA_PROBE(1);
            const uint32_t kb = k_s + sk * L::kTile, qx_s = q_s + X * L::kTile;
            const uint32_t s_t = tmem + (X ? S_COL1 : S_COL0);
#pragma unroll
            for (int kk = 0; kk < D / 16; kk++) {
                const uint32_t off = (kk >> 2) * L::kBox + (kk & 3) * 32;
                mma_f16_ss(s_t, make_sdesc(qx_s + off, hi_k), make_sdesc(kb + off, hi_k), idesc_qk, kk > 0);
            }
            tc_commit(smem_u32(&cb.s_full[X][(t[X] + j) % kRing]));
            FA_PROBE(2);
            return true;
        };
        // O += P V of query tile X for the item's key tile j.
        auto issue_pv = [&](int X, int j) -> bool {
            const int gv = g0 + j, sv = gv % NV;
            if (!mbar_wait(smem_u32(&cb.v_full[sv]), (gv / NV) & 1, ctl, kPVFull)) return false;
            FA_PROBE(3);
            if (!mbar_wait(smem_u32(&cb.p_full[X]), (t[X] + j) & 1, ctl, kPPFull)) return false;
            FA_PROBE(4);
            // the first P V of an item overwrites O: the previous item's epilogue must have read it
            if (j == 0 && itx[X] > 0 && !mbar_wait(smem_u32(&cb.o_free[X]), (itx[X] - 1) & 1, ctl, kPOFree)) return false;
            tc_fence_after();
            FA_PROBE(5);
            const uint32_t vb = v_s + sv * L::kTile;
            const uint32_t p_t = tmem + (X ? P_COL1 : P_COL0), o_t = tmem + (X ? O_COL1 : O_COL0);
#pragma unroll
            for (int kk = 0; kk < kBN / 16; kk++)
                mma_f16_ts(o_t, p_t + kk * 8, make_sdesc(vb + kk * 2048, hi_v), idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
            tc_commit(smem_u32(&cb.pv_done[X][(t[X] + j) % kRing]));
            FA_PROBE(6);
            return true;
        };

        bool ok = true;
        for (int r = 0; ok && r < n_rounds; r++) {
            PairItem it;
            if (!get_pair_item<CAUSAL>(r, n_items, n_bh, n_pairs, seq_len, heads_per_group, it)) continue;
            const int X = warp == kWarpChainA ? 0 : 1;
            const int n_x = X ? it.n_b : it.n_a;
            if (n_x > 0) {
                if (!mbar_wait(smem_u32(&cb.q_full[X]), itx[X] & 1, ctl, kPQFull)) break;
                if (!issue_qk(X, 0)) break;
                for (int j = 0; j < n_x; j++) {
                    if constexpr (INPLACE) {
                        // P(j) lives in the score buffer: Q K^T(j + 1) follows P V(j) in this thread's order
                        if (!issue_pv(X, j)) { ok = false; break; }
                        if (j + 1 < n_x && !issue_qk(X, j + 1)) { ok = false; break; }
                    } else {
                        // the scores of tile j + 1 are produced while tile j is being exponentiated
                        if (j + 1 < n_x && !issue_qk(X, j + 1)) { ok = false; break; }
                        if (!issue_pv(X, j)) { ok = false; break; }
                    }
                }
            }
            t[0] += it.n_a; t[1] += it.n_b;
            itx[0] += 1; itx[1] += it.n_b > 0 ? 1 : 0;
            g0 += it.n;
        }
        FA_PROBE_FLUSH(warp - 7, g0);
        }
        __syncwarp();
    } else if (warp >= 12) {
        // ------------------------------------------------------------ epilogue warps 12-15
        const int r_in_tile = tid - 384;                  // == TMEM lane: (warp & 3) * 32 + lane
        const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
        int n_rv = 0;                                     // rendezvous so far (its parity is the phase to wait for)
        auto rendezvous4 = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&cb.epi));
            const bool w = __all_sync(0xffffffffu, mbar_wait(smem_u32(&cb.epi), n_rv & 1, ctl, kPEpi));
            n_rv++;
            return w;
        };
        int itx[2] = {0, 0}, tx[2] = {0, 0};              // per query tile: items / key tiles so far
        int last_buf = -1;                                // staging tile of the most recent bulk store
        bool ok = true;
        for (int r = 0; ok && r < n_rounds; r++) {
            PairItem it;
            if (!get_pair_item<CAUSAL>(r, n_items, n_bh, n_pairs, seq_len, heads_per_group, it)) continue;
#pragma unroll
            for (int X = 0; X < 2; X++) {
                const int n_x = X ? it.n_b : it.n_a;
                if (n_x == 0) continue;
                tx[X] += n_x;
                const uint32_t t_o = tmem + lane_off + (X ? O_COL1 : O_COL0);
                if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&cb.stats_full[X]), itx[X] & 1, ctl, kPStatsFull))) { ok = false; break; }
                const float inv_l = cb.inv_l[X][r_in_tile];
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&cb.stats_free[X]));
                // O is complete when the item's last P V is
                if (!__all_sync(0xffffffffu, wait_pv_done(X, tx[X] - 1, kPODone))) { ok = false; break; }
                tc_fence_after();
                // the staging tile must have been drained by the bulk store that last read it
                const int buf = (NO == 2) ? X : 0;
                const uint32_t o_sb = o_s + buf * L::kTile;
                if (tid == 384) {
                    if (buf == last_buf) tma_store_wait_read();
                    else tma_store_wait_read_keep1();
                }
                last_buf = buf;
                if (!rendezvous4()) { ok = false; break; }
#pragma unroll 1
                for (int c = 0; c < D / 32; c++) {
                    uint32_t o[32];
                    tmem_ld32_wait(t_o + c * 32, o);
                    if (c == D / 32 - 1) {                // the whole row is out of TMEM: the next item may overwrite O
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&cb.o_free[X]));
                    }
#pragma unroll
                    for (int g8 = 0; g8 < 4; g8++) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; e++)
                            w[e] = pack_16<BF16>(__uint_as_float(o[g8 * 8 + 2 * e]) * inv_l,
                                                 __uint_as_float(o[g8 * 8 + 2 * e + 1]) * inv_l);
                        const int c16 = c * 4 + g8;       // 8-element (16-byte) group index in the row
                        const uint32_t addr = o_sb + (c16 >> 3) * L::kBox + r_in_tile * 128 +
                                              (((c16 & 7) ^ (r_in_tile & 7)) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]),
                                     "r"(w[2]), "r"(w[3]) : "memory");
                    }
                }
                fence_proxy_async_smem();
                if (!rendezvous4()) { ok = false; break; }
                if (tid == 384) {
                    for (int bx = 0; bx < NBOX; bx++)
                        tma_store_3d(&tm_o, o_sb + bx * L::kBox, bx * 64, it.qa + X * kBM, it.bh);
                    tma_store_commit();
                }
                itx[X]++;
            }
        }
        if (tid == 384) tma_store_wait_read();            // the CTA may exit once staging has been read
        __syncwarp();
    } else {
        // ------------------------------------------------------------ softmax of tile X (warps 0-3: A, 4-7: B)
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
        const int X = warp >> 2;
        const int r_in_tile = (warp & 3) * 32 + lane;     // 0..127 == TMEM lane; one thread owns the whole row
        const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t t_s = tmem + lane_off + (X ? S_COL1 : S_COL0);
        const uint32_t t_p = tmem + lane_off + (X ? P_COL1 : P_COL0);
        const uint32_t t_o = tmem + lane_off + (X ? O_COL1 : O_COL0);
        const uint64_t scale2 = pack2(scale_log2, scale_log2);
        int t = 0, itx = 0;                               // key tiles / items of this tile so far
        bool ok = true;
        FA_PROBE_DECL

        for (int r = 0; ok && r < n_rounds; r++) {
            PairItem it;
            if (!get_pair_item<CAUSAL>(r, n_items, n_bh, n_pairs, seq_len, heads_per_group, it)) continue;
            const int n_x = X ? it.n_b : it.n_a;
            if (n_x == 0) continue;
            const int q_start = it.qa + X * kBM;
            const int row = q_start + r_in_tile;
            const int row_limit = CAUSAL ? min(seq_len, row + 1) : seq_len;            // keys [0, row_limit) visible
            const int tile_min_limit = CAUSAL ? min(seq_len, q_start + 1) : seq_len;   // the tile's smallest row_limit
            float m_run = 0.0f;                           // the max in use, in log2 units (set by the first key tile)
            uint64_t lsum2 = pack2(0.0f, 0.0f);

            for (int j = 0; j < n_x; j++, t++) {
                // The votes keep the warp together: every lane leaves the loop or none does.
                if (!__all_sync(0xffffffffu, wait_qk_done(X, t, kPSFull))) { ok = false; break; }
                tc_fence_after();
                FA_PROBE(0);
                uint32_t s[128];
                tmem_ld128_wait(t_s, s);
                FA_PROBE(1);
                if constexpr (!INPLACE) {                 // the scores are in registers: the buffer may be overwritten
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&cb.s_free[X]));
                }
                const int kv_start = j * kBN;
                if ((tile_min_limit - kv_start) < kBN) {  // tile touches the mask or the ragged end
                    const int limit = row_limit - kv_start;   // columns [0,limit) are visible
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
                const bool changed = j > 0 && tile_max > m_run + kRescaleThreshold;
                const float m_new = (j == 0 || changed) ? tile_max : m_run;
                FA_PROBE(2);

                bool pv_waited = INPLACE || t == 0;       // d_head 128: S ready implies the previous P V is done
                // ---- rare: the max in use grew -> rescale O in TMEM before this tile's P V
                if (__any_sync(0xffffffffu, changed)) {
                    if (!pv_waited) {
                        if (!__all_sync(0xffffffffu, wait_pv_done(X, t - 1, kPPvDone))) { ok = false; break; }
                        pv_waited = true;
                    }
                    tc_fence_after();
                    const float factor = changed ? ex2_approx(m_run - m_new) : 1.0f;
                    lsum2 = mul2(lsum2, pack2(factor, factor));
#pragma unroll 1
                    for (int c = 0; c < D / 32; c++) {
                        uint32_t o[32];
                        tmem_ld32_wait(t_o + c * 32, o);
#pragma unroll
                        for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
                        tmem_st_x32(t_o + c * 32, o);
                    }
                    tmem_wait_st();
                }
                m_run = m_new;
                FA_PROBE(3);

                // ---- p = 2^(s*scale*log2e - m); row sum; P -> TMEM as packed 16-bit pairs.  With P in
                // its own columns the stores wait until every exponential is done: by then the P V
                // that reads the previous P has long finished, so the wait below costs nothing.
                const uint64_t negm2 = pack2(-m_new, -m_new);
                uint64_t acc0 = lsum2, acc1 = pack2(0.0f, 0.0f), acc2 = acc1, acc3 = acc1;   // independent sum chains
                constexpr int NCHUNK = 4;                 // P is stored 32 keys at a time
                constexpr int kFirstStoreChunk = INPLACE ? 0 : 1;   // chunks of P held back until the previous P V is done
                constexpr int PAIRS = 64 / NCHUNK;        // 16-bit pairs (TMEM columns of P) per store
                uint32_t pk[64];
#pragma unroll
                for (int c = 0; c < NCHUNK; c++) {
#pragma unroll
                    for (int i = 0; i < PAIRS; i++) {
                        const int e = 2 * (c * PAIRS + i);
                        const uint64_t x = fma2(pack2(__uint_as_float(s[e]), __uint_as_float(s[e + 1])), scale2, negm2);
                        float p0, p1;
                        if (kPolyEvery > 0 && (i % (kPolyEvery > 0 ? kPolyEvery : 1)) == (kPolyEvery > 0 ? kPolyEvery : 1) - 1) {
                            exp2_pair_fma(x, p0, p1);
                        } else {
                            float x0, x1;
                            unpack2(x, x0, x1);
                            p0 = ex2_approx(x0);
                            p1 = ex2_approx(x1);
                        }
                        const uint64_t pp = pack2(p0, p1);
                        if ((i & 3) == 0) acc0 = add2(acc0, pp);
                        else if ((i & 3) == 1) acc1 = add2(acc1, pp);
                        else if ((i & 3) == 2) acc2 = add2(acc2, pp);
                        else acc3 = add2(acc3, pp);
                        pk[c * PAIRS + i] = pack_16<BF16>(p0, p1);
                    }
                    if (c == kFirstStoreChunk && !pv_waited) {
                        // P has its own columns: the P V that read the previous P must be done before
                        // they change.  The first chunks of P stay in registers meanwhile.
                        if (!__all_sync(0xffffffffu, wait_pv_done(X, t - 1, kPPvDone))) { ok = false; break; }
                        tc_fence_after();
                        pv_waited = true;
                    }
                    if (c >= kFirstStoreChunk) {
                        if (c == kFirstStoreChunk) {
#pragma unroll
                            for (int c2 = 0; c2 < kFirstStoreChunk; c2++)
                                tmem_st_x16(t_p + c2 * PAIRS, *reinterpret_cast<uint32_t (*)[16]>(&pk[c2 * PAIRS]));
                        }
                        tmem_st_x16(t_p + c * PAIRS, *reinterpret_cast<uint32_t (*)[16]>(&pk[c * PAIRS]));
                    }
                }
                if (!ok) break;
                lsum2 = add2(add2(acc0, acc1), add2(acc2, acc3));
                FA_PROBE(4);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&cb.p_full[X]));
                FA_PROBE(5);
            }
            if (!ok) break;

            // ---- end of the item: LSE, and 1 / row sum for the epilogue warps
            float l0, l1;
            unpack2(lsum2, l0, l1);
            const float l_run = l0 + l1;
            if (lse_out != nullptr && row < seq_len)
                lse_out[static_cast<size_t>(it.bh) * seq_len + row] = kLn2 * (m_run + log2f(l_run));
            if (itx > 0 &&
                !__all_sync(0xffffffffu, mbar_wait(smem_u32(&cb.stats_free[X]), (itx - 1) & 1, ctl, kPStatsFree))) break;
            cb.inv_l[X][r_in_tile] = 1.0f / l_run;
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&cb.stats_full[X]));
            itx++;
            FA_PROBE(6);
        }
        if ((warp & 3) == 0) FA_PROBE_FLUSH(X, t);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem, TMEM_COLS);
}

template <int D, bool CAUSAL, bool BF16>
int launch_pair_instance(const fa_prefill_args& a, DeviceState* st, int heads_per_group, const CUtensorMap& tq,
                         const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to) {
    using L = PairSmem<D>;
    auto kernel = prefill_pair_kernel<D, CAUSAL, BF16>;
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
    const unsigned grid = (unsigned)(n_items < st->sm_count ? n_items : st->sm_count);
    kernel<<<grid, kThreads, L::kTotal, static_cast<cudaStream_t>(a.stream)>>>(
        tq, tk, tv, to, a.lse, a.seq_len, n_bh, n_pairs, (int)n_items, heads_per_group, a.scale * kLog2e, st->status);
    FA_CUDA_TRY(cudaGetLastError());
    return FA_OK;
}

}  // namespace

int launch_prefill_pair_16bit(const fa_prefill_args& a, DeviceState* st, int heads_per_group, const CUtensorMap& tq,
                              const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to) {
    const bool bf = a.dtype == FA_DTYPE_BF16;
    const bool causal = a.causal != 0;
#define FA_DISPATCH(DH)                                                                               \
    (causal ? (bf ? launch_pair_instance<DH, true, true>(a, st, heads_per_group, tq, tk, tv, to)      \
                  : launch_pair_instance<DH, true, false>(a, st, heads_per_group, tq, tk, tv, to))    \
            : (bf ? launch_pair_instance<DH, false, true>(a, st, heads_per_group, tq, tk, tv, to)     \
                  : launch_pair_instance<DH, false, false>(a, st, heads_per_group, tq, tk, tv, to)))
    if (a.d_head == 64) return FA_DISPATCH(64);
    return FA_DISPATCH(128);
#undef FA_DISPATCH
}

}  // namespace fa
