// Prefill forward kernel for sm_100a: fp16 / bf16 / e4m3 inputs, d_head 64 or
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
// Persistent kernel: one CTA of 16 warps per SM walks a list of work items (one
// 128-row query tile of one (batch, head) each), heaviest first under the causal
// mask, dealt to the CTAs in boustrophedon order so the per-CTA totals even out.
//
//   warps 8, 11        TMA producers (one lane each): Q per item and the K tiles / the V
//   (one lane each)    tiles (128 keys) through mbarrier-guarded shared-memory rings,
//                      128-byte swizzle.  K and V have a producer each so that K loads
//                      are not held back behind the later-freed V slots.
//   warp 9             issues S = Q K^T (tcgen05.mma, lane 0) into one of THREE score
//                      buffers in TMEM, used round-robin; it waits for the tile's K and
//                      for the P V that last read the buffer (three tiles back).
//   warp 10            issues O += P V: P from TMEM, V (MN-major) from shared memory.
//                      Q K^T and P V have an issuer each because every tcgen05.mma /
//                      commit costs its issuing thread ~50-100 clocks; one thread doing
//                      both was the bottleneck.  Each issuer commits once per tile, onto a
//                      ring of completion barriers that every interested party waits on
//                      (softmax: S is there; K producer: slot free / Q K^T issuer: score
//                      buffer free; V producer: slot free; softmax: O may be rescaled).
//   warps 0-7          softmax, two groups of four warps.  Group 0 owns the even key
//                      tiles, group 1 the odd ones, so the two groups are in different
//                      phases of their tiles and share the MUFU pipe.  A thread owns a
//                      whole query row (TMEM lane) of its tiles: one tcgen05.ld brings the
//                      128 scores into registers, no cross-thread reduction; p =
//                      2^(s*scale*log2e - m) with packed f32x2 arithmetic; P goes back to
//                      TMEM as 16-bit pairs IN PLACE, over the first 64 columns of the
//                      scores it came from, so the softmax never waits for a P buffer.
//                      The max in use is handed from tile to tile through tagged
//                      shared-memory slots; it only moves (and O is only rescaled, in
//                      TMEM) when a tile's max exceeds it by more than 2^8.  At the end of
//                      an item the two threads of a row leave (max, partial sum) for the
//                      epilogue and go straight on to the next item.
//   warps 12-15        epilogue of every item, one thread per query row: combine the two
//                      partial sums, O / l -> 16-bit -> swizzled staging -> TMA store
//                      (clipped per head); LSE as fp32.  The tensor pipe and the softmax
//                      already work on the next item meanwhile.  In decode over an e4m3
//                      cache the same warps first turn each V tile into the fp16 operand
//                      of P V (the e4m3 prefill gets an fp16 V from a pre-pass instead).
//
// TMEM (all 512 columns): three score buffers [0,128) [128,256) [256,384), O [384,384+D).
#include <atomic>
#include <cmath>

#include "host_common.h"
#include "ptx.cuh"
#include "tmem_ld.cuh"

namespace fa {
namespace {

constexpr int kBM = 128;                 // query rows per work item
constexpr int kBN = 128;                 // keys per tile
constexpr int kThreads = 512;            // 16 warps: 0-7 softmax, 8 and 11 TMA, 9 Q K^T issuer, 10 P V issuer, 12-15 epilogue (+ e4m3 V conversion)
// setmaxnreg moves registers inside the pool the CTA got at launch (threads x registers at launch,
// not the whole register file): an increase beyond that pool blocks forever.
constexpr int kRegsLaunch = (65536 / kThreads) / 8 * 8;   // 128 at 512 threads (what __launch_bounds__ yields)
constexpr int kRegsSoftmax = 192;        // warps 0-7
constexpr int kRegsOther = 64;           // warps 8-11
constexpr int kRegsHelper = 64;          // warps 12-15
static_assert(256 * kRegsSoftmax + 128 * kRegsOther + 128 * kRegsHelper <= kThreads * kRegsLaunch,
              "setmaxnreg targets exceed the CTA's register pool");
constexpr int kNU = 3;                   // score buffers in TMEM (S, then P in place), used round-robin
constexpr int kRing = 4;                 // entries of the Q K^T / P V completion rings
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;   // log2 units: rescale only if max grew > 2^8
#ifndef FA_GROUP_MB
#define FA_GROUP_MB 16
#endif

// Barrier ids reported in the status word when a wait gives up.
enum : int { kBarQFull = 1, kBarQEmpty = 2, kBarKFull = 3, kBarKEmpty = 4, kBarVFull = 5,
             kBarVEmpty = 6, kBarSFull = 7, kBarSFree = 8, kBarPFull = 9, kBarPV = 10,
             kBarOFree = 11, kBarV8Full = 12, kBarV8Empty = 13, kBarM = 14, kBarEpi = 15, kBarODone = 16, kBarStats = 17, kBarStatsFree = 18 };

// Two e4m3 codes -> two fp16 values (exact).
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint16_t v) {
    uint32_t r;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
    return r;
}


template <int D, bool FP8, bool V8 = FP8>
struct PrefillSmem {
    static constexpr int kNBox    = D / 64;               // 64-column (128-byte) boxes per 16-bit row
    static constexpr int kBox     = 128 * 128;            // one box: 128 rows x 128 bytes
    // e4m3 rows of d_head 128 are exactly one 128-byte box.
    static constexpr int kQBytes  = FP8 ? kBox : kNBox * kBox;
    static constexpr int kKBytes  = kQBytes;
    static constexpr int kVBytes  = kNBox * kBox;         // 16-bit V operand of P V (e4m3: converted copy)
    static constexpr int kV8Bytes = V8 ? kBox : 0;       // landing buffers of the e4m3 V tiles
    static constexpr int kOBytes  = kNBox * kBox;         // epilogue staging (16-bit output tile)
    static constexpr int NK  = (D == 64) ? 4 : 2;
    static constexpr int NV  = (D == 64) ? 4 : (V8 ? 3 : 2);   // e4m3: the converted (fp16) V tiles
    static constexpr int NV8 = V8 ? 2 : 0;
    static constexpr int kTotal = kQBytes + NK * kKBytes + NV * kVBytes + NV8 * kV8Bytes + kOBytes + 1024;
};

// Grouped-query decode mode (device side of GqaLaunch).
struct GqaDev {
    float* o_part;          // [row][split][D] fp32, row = (batch * n_tok + token) * Hq + query head
    float* lse_part;        // [row][split]
    uint16_t* o_final;      // with one split the epilogue writes the 16-bit result and its LSE directly
    float* lse_final;       // (may be null)
    int n_splits, tiles_per_split, group, n_hkv;
    int n_tok;              // query tokens per sequence
    int tok_per_tile;       // tokens per query tile (row r of a tile: token r / group, head r % group)
    int n_qt;               // query tiles per (batch, KV head) = ceil(n_tok / tok_per_tile)
    int live_rows;          // rows of a tile a Q load writes = min(tok_per_tile, n_tok) * group
    const int* seq_lens;    // per-sequence KV lengths, or null: every sequence has seq_len keys
    const int* block_table; // paged cache: [batch][table_stride] page numbers, or null
    int table_stride;
    int page_shift;         // log2(page size)
};

// Work list: item index -> (query tile, head), heaviest first when causal.  In grouped-query
// decode mode an item is (batch x KV head, query tile, KV split): key tiles [t0, t0 + n_kv) of that
// head for the tokens from tok0 on.
struct Item { int q_start, bh, n_kv, t0, split, kv_len, tok0; bool empty; };

// Index of the partial result of tile row r: output row ((batch * n_tok + token) * Hq + query head),
// then the KV split.
__device__ __forceinline__ size_t gqa_partial_index(const GqaDev& gq, const Item& it, int r) {
    const int b = it.bh / gq.n_hkv, hkv = it.bh - b * gq.n_hkv;
    const int tl = r / gq.group, g = r - tl * gq.group;
    const size_t row = (static_cast<size_t>(b) * gq.n_tok + it.tok0 + tl) * (gq.n_hkv * gq.group) + hkv * gq.group + g;
    return row * gq.n_splits + it.split;
}

template <bool CAUSAL, bool GQA, bool GROUPED>
__device__ __forceinline__ bool get_item(int k, int n_items, int n_bh, int n_qtiles, int seq_len,
                                         const GqaDev& gq, Item& it) {
    const int G = gridDim.x, c = blockIdx.x;
    if constexpr (GQA) {
        const int idx = k * G + c;                    // items are (nearly) equal: plain round-robin
        it.empty = false;
        if (idx >= n_items) return false;
        const int bq = idx / gq.n_splits;             // (batch x KV head, query tile)
        it.split = idx - bq * gq.n_splits;
        // the later query tiles see more keys: all heads' last tiles first
        const int qt_rev = bq / n_bh;
        it.bh = bq - qt_rev * n_bh;
        it.tok0 = (gq.n_qt - 1 - qt_rev) * gq.tok_per_tile;
        it.t0 = it.split * gq.tiles_per_split;
        it.kv_len = gq.seq_lens ? min(seq_len, max(0, __ldg(gq.seq_lens + it.bh / gq.n_hkv))) : seq_len;
        // keys the tile's last token sees (the query tokens are the last n_tok entries of the cache)
        const int kv_vis = min(it.kv_len, it.kv_len - gq.n_tok + min(gq.n_tok, it.tok0 + gq.tok_per_tile));
        it.n_kv = min(gq.tiles_per_split, (max(kv_vis, 0) + kBN - 1) / kBN - it.t0);
        it.q_start = 0;
        // a split that lies wholly past the end of a short sequence: no role touches it, the
        // epilogue warps only record an empty partial
        it.empty = it.n_kv <= 0;
        return !it.empty;
    }
    it.t0 = 0;
    it.split = 0;
    it.kv_len = seq_len;
    it.tok0 = 0;
    it.empty = false;
    const int idx = (k & 1) ? k * G + (G - 1 - c) : k * G + c;     // boustrophedon deal
    if (idx >= n_items) return false;
    // GROUPED: heads are taken in groups of gq.group (reused here as "heads per group"); within a
    // group the list runs query tile by query tile over the group's heads, so the K and V that the
    // CTAs stream at any one time belong to one group and stay in L2.  A separate instance, because
    // the extra index arithmetic (and the code it adds to every role) costs short work items 4-6 %.
    int qrank;
    if constexpr (GROUPED) {
        const int per_group = gq.group * n_qtiles;
        const int gi = idx / per_group, rem = idx - gi * per_group;
        const int h0 = gi * gq.group, hin = min(gq.group, n_bh - h0);
        qrank = rem / hin;
        it.bh = h0 + rem - qrank * hin;
        // Under the causal mask every group runs from its heaviest to its lightest tiles, a sawtooth
        // that the boustrophedon deal balances poorly (per-CTA totals up to 6 % above the mean on 32
        // heads of 64 tiles); odd groups run light to heavy instead, which halves that (a CTA's total
        // does not depend on the order in which it meets its items).
        if (CAUSAL && (gi & 1)) qrank = n_qtiles - 1 - qrank;
    } else {
        qrank = idx / n_bh;
        it.bh = idx % n_bh;
    }
    const int qt = CAUSAL ? (n_qtiles - 1 - qrank) : qrank;
    it.q_start = qt * kBM;
    const int kv_len = CAUSAL ? min(seq_len, it.q_start + kBM) : seq_len;
    it.n_kv = (kv_len + kBN - 1) / kBN;
    return true;
}

// FP8: Q, K, V are e4m3 codes with per-head scales.  S = Q K^T runs on the 8-bit tensor-core
// kind; P V runs on the 16-bit kind with P in fp16, because an e4m3 P (3 mantissa bits) misses
// the output tolerance, so V has to be fp16 as well (exact).  Prefill gets it from a pre-pass
// over the whole tensor (e4m3_to_f16_kernel) and loads it like any 16-bit V; decode over an
// e4m3 cache (GQA) cannot rewrite the cache, so there the e4m3 V tiles land in buffers of
// their own and warps 12-15 convert each one in shared memory (V8).
// The Q and K scales fold into the softmax scale, the V scale into the final normalisation;
// the output is bf16.
template <int D, bool CAUSAL, bool BF16, bool FP8, bool GQA, bool GROUPED>
__global__ void __launch_bounds__(kThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
               float* __restrict__ lse_out, int seq_len, int n_bh, int n_qtiles, int n_items,
               float scale_log2_in, const float* __restrict__ q_scale,
               const float* __restrict__ k_scale, const float* __restrict__ v_scale, int* status,
               const GqaDev gq) {
    static_assert(!FP8 || (D == 128 && BF16), "e4m3 variant: d_head 128, bf16 output");
    static_assert(!GQA || !CAUSAL, "grouped-query decode: one query row per head, every key visible");
    constexpr bool V8 = FP8 && GQA;                       // V arrives as e4m3 and is converted in shared memory
    using L = PrefillSmem<D, FP8, V8>;
    constexpr int NBOX = L::kNBox, NK = L::NK, NV = L::NV;
    constexpr uint32_t O_COL = kNU * 128;
    static_assert(NK <= kRing && NV <= kRing && kNU <= kRing, "a ring entry must not be reused before its waiters have looked");
    static_assert(O_COL + D <= 512, "TMEM columns");
    constexpr uint32_t TMEM_COLS = 512;
    constexpr bool P_BF16 = BF16 && !FP8;                 // type of P (and of the V operand of P V)
    constexpr uint32_t FMT = P_BF16 ? kFmtBF16 : kFmtF16;

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_qf, bar_qe, bar_ofree, bar_odone;
    __shared__ __align__(8) uint64_t bar_kf[NK], bar_vf[NV];
    // completion rings of the two MMA streams: Q K^T / P V of tile g arrive on entry g % kRing
    __shared__ __align__(8) uint64_t bar_qk[kRing], bar_pvd[kRing];
    __shared__ __align__(8) uint64_t bar_pf[kNU];            // P of the tile in score buffer u is in TMEM
    __shared__ __align__(8) uint64_t bar_v8f[2], bar_v8e[2];
    __shared__ __align__(8) uint64_t bar_epi;                // rendezvous of the warps that run the epilogue
    __shared__ __align__(8) uint64_t bar_vraw;               // grouped-query decode: a V tile that still needs its tail rows cleared
    // per item parity and row: {max in use (float bits), index of the tile it was decided for};
    // written with one 8-byte store by the tile's owner, polled by the owner of the next tile
    __shared__ __align__(8) uint2 m_slot[2][128];
    // per item parity, group and row: final reference max and partial row sum of a softmax thread
    __shared__ float xm[2][2][128], xsum[2][2][128];
    __shared__ __align__(8) uint64_t bar_stats[2], bar_stats_free[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_s = base;
    const uint32_t k_s = q_s + L::kQBytes;
    const uint32_t v_s = k_s + NK * L::kKBytes;
    const uint32_t v8_s = v_s + NV * L::kVBytes;
    const uint32_t o_s = v8_s + L::NV8 * L::kV8Bytes;
    WaitCtl ctl{&abort_flag, status};

    if (tid == 0) {
        mbar_init(smem_u32(&bar_qf), 1);
        mbar_init(smem_u32(&bar_qe), 1);
        mbar_init(smem_u32(&bar_ofree), 4);              // the epilogue warps have read O
        mbar_init(smem_u32(&bar_odone), 1);
        for (int i = 0; i < NK; i++) mbar_init(smem_u32(&bar_kf[i]), 1);
        for (int i = 0; i < NV; i++) mbar_init(smem_u32(&bar_vf[i]), V8 ? 128 : 1);
        for (int i = 0; i < kRing; i++) { mbar_init(smem_u32(&bar_qk[i]), 1); mbar_init(smem_u32(&bar_pvd[i]), 1); }
        for (int i = 0; i < kNU; i++) mbar_init(smem_u32(&bar_pf[i]), 4);   // one arrival per warp of the owning group
        for (int i = 0; i < 2; i++) {
            mbar_init(smem_u32(&bar_v8f[i]), 1);
            mbar_init(smem_u32(&bar_v8e[i]), 128);
        }
        mbar_init(smem_u32(&bar_epi), 4);
        mbar_init(smem_u32(&bar_vraw), 1);
        for (int i = 0; i < 2; i++) { mbar_init(smem_u32(&bar_stats[i]), 8); mbar_init(smem_u32(&bar_stats_free[i]), 4); }
        abort_flag = 0;
        fence_mbar_init();
    }
    if (tid < 256) m_slot[tid >> 7][tid & 127] = make_uint2(0u, 0xFFFFFFFFu);   // no tile has this index
    if constexpr (GQA) {
        // decode: a Q load only writes the rows that carry a (token, head) pair; the other rows of the
        // query tile are zero for the whole launch
        for (int i = tid; i < L::kQBytes / 16; i += kThreads)
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(q_s + i * 16), "r"(0u) : "memory");
        fence_proxy_async_smem();
    }
    if (warp == 8 && lane == 0) {
        prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v); prefetch_tensormap(&tm_o);
    }
    __syncthreads();
    if (warp == 9) tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const int n_rounds = (n_items + gridDim.x - 1) / gridDim.x;

    // Grouped-query decode: one 128-key tile of K or V of (batch, KV head) from the cache.  Dense or
    // strided cache: tensor map (d, key, KV head, batch).  Paged cache: tensor map (d, key in page,
    // KV head, page); a tile is one box inside a page, or 128 / page_size boxes of one page each;
    // pages past the end of the sequence are fetched at coordinate -1, which reads as zero.
    auto load_cache_tile = [&](uint32_t dst, const CUtensorMap* tm, uint32_t bar, const Item& it, int j) {
        constexpr int NB = FP8 ? 1 : NBOX;            // boxes per tile row: e4m3 rows are one 128-byte box
        constexpr int XS = FP8 ? 128 : 64;            // elements per box row
        const int hkv = it.bh % gq.n_hkv, b = it.bh / gq.n_hkv;
        const int r0 = (it.t0 + j) * kBN;
        if (gq.block_table == nullptr) {
            for (int bx = 0; bx < NB; bx++) tma_load_4d(dst + bx * L::kBox, tm, bar, bx * XS, r0, hkv, b);
        } else {
            const int ps = 1 << gq.page_shift;
            const int rows = min(ps, kBN);            // rows per box
            const int* tbl = gq.block_table + static_cast<size_t>(b) * gq.table_stride;
            for (int i = 0; i < kBN / rows; i++) {
                const int rr = r0 + i * rows;
                const int page = rr < it.kv_len ? __ldg(tbl + (rr >> gq.page_shift)) : -1;
                for (int bx = 0; bx < NB; bx++)
                    tma_load_4d(dst + bx * L::kBox + i * rows * 128, tm, bar, bx * XS, rr & (ps - 1), hkv, page);
            }
        }
    };
    if (warp >= 12) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsHelper));
    else if (warp >= 8) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
    if (warp == 8) {
        // ------------------------------------------------------------ TMA producer: Q and K
        // (K and V have a producer each: a K slot frees when its Q K^T is done, a V slot only when
        // its P V is done, much later; one in-order producer would hold K loads back behind V.)
        if (lane == 0) {
            constexpr int NLOAD = FP8 ? 1 : NBOX;         // boxes per Q / K tile
            constexpr int XSTEP = FP8 ? 128 : 64;         // elements per box row
            int g = 0, it_n = 0;
            bool ok = true;
            for (int r = 0; ok && r < n_rounds; r++) {
                Item it;
                if (!get_item<CAUSAL, GQA, GROUPED>(r, n_items, n_bh, n_qtiles, seq_len, gq, it)) continue;
                if (it_n > 0 && !mbar_wait(smem_u32(&bar_qe), (it_n - 1) & 1, ctl, kBarQEmpty)) break;
                if constexpr (GQA) {
                    // the box holds only the live rows (token-major); the rest of the tile stays zero
                    mbar_arrive_expect_tx(smem_u32(&bar_qf), NLOAD * gq.live_rows * 128);
                    for (int b = 0; b < NLOAD; b++)
                        tma_load_5d(q_s + b * L::kBox, &tm_q, smem_u32(&bar_qf), b * XSTEP, 0, it.tok0, it.bh % gq.n_hkv,
                                    it.bh / gq.n_hkv);
                } else {
                    mbar_arrive_expect_tx(smem_u32(&bar_qf), L::kQBytes);
                    for (int b = 0; b < NLOAD; b++)
                        tma_load_3d(q_s + b * L::kBox, &tm_q, smem_u32(&bar_qf), b * XSTEP, it.q_start, it.bh);
                }
                for (int j = 0; j < it.n_kv; j++, g++) {
                    const int sk = g % NK;
                    // the slot was last read by Q K^T of tile g - NK
                    if (g >= NK && !mbar_wait(smem_u32(&bar_qk[(g - NK) % kRing]), ((g - NK) / kRing) & 1, ctl, kBarKEmpty)) { ok = false; break; }
                    mbar_arrive_expect_tx(smem_u32(&bar_kf[sk]), L::kKBytes);
                    if constexpr (GQA) {
                        load_cache_tile(k_s + sk * L::kKBytes, &tm_k, smem_u32(&bar_kf[sk]), it, j);
                    } else {
                        for (int b = 0; b < NLOAD; b++)
                            tma_load_3d(k_s + sk * L::kKBytes + b * L::kBox, &tm_k, smem_u32(&bar_kf[sk]),
                                        b * XSTEP, j * kBN, it.bh);
                    }
                }
                it_n++;
            }
        }
        __syncwarp();
    } else if (warp == 11) {
        // ------------------------------------------------------------ TMA producer: V
        if (lane == 0) {
            int g = 0, n_scrub = 0;
            bool ok = true;
            for (int r = 0; ok && r < n_rounds; r++) {
                Item it;
                if (!get_item<CAUSAL, GQA, GROUPED>(r, n_items, n_bh, n_qtiles, seq_len, gq, it)) continue;
                for (int j = 0; j < it.n_kv; j++, g++) {
                    if constexpr (V8) {
                        // e4m3 V lands in its own buffers; warps 12-15 turn it into the fp16 operand.
                        const int s8 = g & 1;
                        if (g >= 2 && !mbar_wait(smem_u32(&bar_v8e[s8]), ((g >> 1) - 1) & 1, ctl, kBarV8Empty)) { ok = false; break; }
                        mbar_arrive_expect_tx(smem_u32(&bar_v8f[s8]), L::kV8Bytes);
                        if constexpr (GQA)
                            load_cache_tile(v8_s + s8 * L::kV8Bytes, &tm_v, smem_u32(&bar_v8f[s8]), it, j);
                        else
                            tma_load_3d(v8_s + s8 * L::kV8Bytes, &tm_v, smem_u32(&bar_v8f[s8]), 0, j * kBN, it.bh);
                    } else {
                        const int sv = g % NV;
                        // the slot was last read by P V of tile g - NV
                        if (g >= NV && !mbar_wait(smem_u32(&bar_pvd[(g - NV) % kRing]), ((g - NV) / kRing) & 1, ctl, kBarVEmpty)) { ok = false; break; }
                        if constexpr (GQA) {
                            // Rows of the sequence's last tile past its end are stale cache contents when the
                            // cache is paged or longer than the sequence (a dense cache reads them as zero).
                            // P is exactly 0 there, but 0 x NaN would still poison O, so those rows of V are
                            // cleared before the P V issuer may see the tile: the load completes on a private
                            // barrier, this thread clears the rows and then releases the tile itself.
                            const int valid = it.kv_len - (it.t0 + j) * kBN;      // rows of this tile inside the sequence
                            const bool scrub = valid < kBN && (gq.seq_lens != nullptr || gq.block_table != nullptr);
                            const uint32_t vdst = v_s + sv * L::kVBytes;
                            if (!scrub) {
                                mbar_arrive_expect_tx(smem_u32(&bar_vf[sv]), L::kVBytes);
                                load_cache_tile(vdst, &tm_v, smem_u32(&bar_vf[sv]), it, j);
                            } else {
                                mbar_arrive_expect_tx(smem_u32(&bar_vraw), L::kVBytes);
                                load_cache_tile(vdst, &tm_v, smem_u32(&bar_vraw), it, j);
                                if (!mbar_wait(smem_u32(&bar_vraw), n_scrub & 1, ctl, kBarVFull)) { ok = false; break; }
                                n_scrub++;
                                for (int row = valid; row < kBN; row++)
                                    for (int b = 0; b < NBOX; b++)
                                        for (int q16 = 0; q16 < 8; q16++)
                                            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(
                                                vdst + b * L::kBox + row * 128 + q16 * 16), "r"(0u) : "memory");
                                fence_proxy_async_smem();
                                mbar_arrive(smem_u32(&bar_vf[sv]));
                            }
                        } else {
                            mbar_arrive_expect_tx(smem_u32(&bar_vf[sv]), L::kVBytes);
                            for (int b = 0; b < NBOX; b++)
                                tma_load_3d(v_s + sv * L::kVBytes + b * L::kBox, &tm_v, smem_u32(&bar_vf[sv]),
                                            b * 64, j * kBN, it.bh);
                        }
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 9) {
        // ------------------------------------------------------------ Q K^T issuer
        // The whole warp walks the loop (uniform control flow keeps the descriptors in uniform
        // registers); lane 0 issues.  A tcgen05.mma or commit costs the issuing thread ~50 clocks,
        // so Q K^T and P V have an issuer warp each: this one never waits for the softmax of a
        // tile, only for its score buffer to be handed back.
        constexpr uint32_t QKFMT = FP8 ? kFmtE4M3 : FMT;
        constexpr uint32_t idesc_qk = make_idesc(kBM, kBN, QKFMT, QKFMT, kMajorK, kMajorK);
        constexpr uint64_t hi_k = make_sdesc_hi(16, 1024);
        int g = 0, it_n = 0, u = 0;                       // u == g % kNU: the tile's score buffer
        bool ok = true;
        for (int r = 0; ok && r < n_rounds; r++) {
            Item it;
            if (!get_item<CAUSAL, GQA, GROUPED>(r, n_items, n_bh, n_qtiles, seq_len, gq, it)) continue;
            if (!mbar_wait(smem_u32(&bar_qf), it_n & 1, ctl, kBarQFull)) break;
            for (int j = 0; j < it.n_kv; j++, g++) {
                const int sk = g % NK;
                if (!mbar_wait(smem_u32(&bar_kf[sk]), (g / NK) & 1, ctl, kBarKFull)) { ok = false; break; }
                // the score buffer last held S and then P of tile g - kNU: that P V must be done
                if (g >= kNU && !mbar_wait(smem_u32(&bar_pvd[(g - kNU) % kRing]), ((g - kNU) / kRing) & 1, ctl, kBarSFree)) { ok = false; break; }
                tc_fence_after();
                const uint32_t kb = k_s + sk * L::kKBytes;
                const uint32_t sc = tmem + u * 128;
                if constexpr (FP8) {
#pragma unroll
                    for (int kk = 0; kk < D / 32; kk++) {         // 32 e4m3 (32 bytes) of d_head per MMA
                        const uint64_t da = make_sdesc(q_s + kk * 32, hi_k), db = make_sdesc(kb + kk * 32, hi_k);
                        if (lane == 0) mma_f8_ss(sc, da, db, idesc_qk, kk > 0);
                    }
                } else {
#pragma unroll
                    for (int kk = 0; kk < D / 16; kk++) {
                        const uint32_t off = (kk >> 2) * L::kBox + (kk & 3) * 32;
                        const uint64_t da = make_sdesc(q_s + off, hi_k), db = make_sdesc(kb + off, hi_k);
                        if (lane == 0) mma_f16_ss(sc, da, db, idesc_qk, kk > 0);
                    }
                }
                if (lane == 0) {
                    tc_commit(smem_u32(&bar_qk[g % kRing]));                // S is ready; the K slot is free
                    if (j == it.n_kv - 1) tc_commit(smem_u32(&bar_qe));   // Q is dead after the item's last Q K^T
                }
                __syncwarp();
                u = (u == kNU - 1) ? 0 : u + 1;
            }
            it_n++;
        }
    } else if (warp == 10) {
        // ------------------------------------------------------------ P V issuer
        constexpr uint32_t idesc_pv = make_idesc(kBM, D, FMT, FMT, kMajorK, kMajorMN);
        constexpr uint64_t hi_v = make_sdesc_hi(L::kBox, 1024);
        int g = 0, it_n = 0, u = 0, u_phase = 0;          // u == g % kNU, u_phase == (g / kNU) & 1
        bool ok = true;
        for (int r = 0; ok && r < n_rounds; r++) {
            Item it;
            if (!get_item<CAUSAL, GQA, GROUPED>(r, n_items, n_bh, n_qtiles, seq_len, gq, it)) continue;
            for (int j = 0; j < it.n_kv; j++, g++) {
                const int sv = g % NV;
                if (!mbar_wait(smem_u32(&bar_vf[sv]), (g / NV) & 1, ctl, kBarVFull)) { ok = false; break; }
                if (!mbar_wait(smem_u32(&bar_pf[u]), u_phase, ctl, kBarPFull)) { ok = false; break; }
                // the first P V of an item overwrites O: the previous item's epilogue must have read it
                if (j == 0 && it_n > 0 && !mbar_wait(smem_u32(&bar_ofree), (it_n - 1) & 1, ctl, kBarOFree)) { ok = false; break; }
                tc_fence_after();
                const uint32_t vb = v_s + sv * L::kVBytes;
                const uint32_t pc = tmem + u * 128;         // P overwrote the first 64 columns of the tile's S
#pragma unroll
                for (int kk = 0; kk < kBN / 16; kk++) {
                    const uint64_t db = make_sdesc(vb + kk * 2048, hi_v);
                    if (lane == 0) mma_f16_ts(tmem + O_COL, pc + kk * 8, db, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                }
                if (lane == 0) {
                    tc_commit(smem_u32(&bar_pvd[g % kRing]));               // score buffer and V slot are free
                    if (j == it.n_kv - 1) tc_commit(smem_u32(&bar_odone));   // the item's O is complete
                }
                __syncwarp();
                if (u == kNU - 1) { u = 0; u_phase ^= 1; } else { u++; }
            }
            it_n++;
        }
    } else if (warp >= 12) {
        // ------------------------------------------------------------ helper warps 12-15
        // Epilogue of every item, one thread per query row: combine the two softmax threads'
        // (max, sum), read the row of O from TMEM, normalise, stage in swizzled shared memory,
        // TMA-store; the softmax warps are already on the next item.  In decode over an e4m3 cache
        // (V8) the same warps first turn each V tile of the item into the fp16 operand of P V.
        const int ct = tid - 384;                         // 0..127
        const int r_in_tile = ct;                         // == TMEM lane: (warp & 3) * 32 + lane
        const uint32_t t_o = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + O_COL;
        auto rendezvous4 = [&](uint32_t parity) -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_epi));
            return __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_epi), parity, ctl, kBarEpi));
        };
        int it_n = 0, g = 0;
        bool ok = true;
        for (int r = 0; ok && r < n_rounds; r++) {
            Item it;
            if (!get_item<CAUSAL, GQA, GROUPED>(r, n_items, n_bh, n_qtiles, seq_len, gq, it)) {
                if constexpr (GQA) {
                    // a KV split past the end of a short sequence: weight zero in the merge
                    if (it.empty && r_in_tile < gq.live_rows && it.tok0 + r_in_tile / gq.group < gq.n_tok) {
                        const size_t pidx = gqa_partial_index(gq, it, r_in_tile);
                        if (gq.n_splits == 1) {               // the only split of a sequence without keys: O = 0
                            uint4* dst = reinterpret_cast<uint4*>(gq.o_final + pidx * D);
                            for (int e = 0; e < D / 8; e++) dst[e] = make_uint4(0u, 0u, 0u, 0u);
                            if (gq.lse_final != nullptr) gq.lse_final[pidx] = -INFINITY;
                        } else {
                            gq.lse_part[pidx] = -INFINITY;
                            float4* dst = reinterpret_cast<float4*>(gq.o_part + pidx * D);
                            for (int e = 0; e < D / 4; e++) dst[e] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                        }
                    }
                }
                continue;
            }
            if constexpr (V8) {
                // ---- e4m3 -> fp16 conversion of the item's V tiles (exact)
                for (int j = 0; j < it.n_kv; j++, g++) {
                    const int s8 = g & 1, sv = g % NV;
                    bool w = mbar_wait(smem_u32(&bar_v8f[s8]), (g >> 1) & 1, ctl, kBarV8Full);
                    // the fp16 buffer must have been consumed by the P V that last read it
                    if (g >= NV) w = w && mbar_wait(smem_u32(&bar_pvd[(g - NV) % kRing]), ((g - NV) / kRing) & 1, ctl, kBarVEmpty);
                    if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
                    const uint32_t src_base = v8_s + s8 * L::kV8Bytes;
                    const uint32_t dst_base = v_s + sv * L::kVBytes;
                    // decode over a cache: rows past the sequence's end may hold stale bytes (NaN codes
                    // included); they are written as zero so that P = 0 there cannot poison O
                    const int valid = GQA ? it.kv_len - (it.t0 + j) * kBN : kBN;
#pragma unroll 4
                    for (int i = 0; i < (kBN * 16) / 128; i++) {
                        const int c16 = ct + i * 128;         // 8-element group: row c16/16, group-in-row c16%16
                        const int rr = c16 >> 4, c8 = c16 & 15;
                        const uint32_t src = src_base + rr * 128 + (((c8 >> 1) ^ (rr & 7)) << 4) + ((c8 & 1) << 3);
                        uint32_t lo, hi;
                        asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "r"(src));
                        if (GQA && rr >= valid) { lo = 0u; hi = 0u; }
                        const uint32_t w0 = e4m3x2_to_f16x2(static_cast<uint16_t>(lo & 0xFFFFu));
                        const uint32_t w1 = e4m3x2_to_f16x2(static_cast<uint16_t>(lo >> 16));
                        const uint32_t w2 = e4m3x2_to_f16x2(static_cast<uint16_t>(hi & 0xFFFFu));
                        const uint32_t w3 = e4m3x2_to_f16x2(static_cast<uint16_t>(hi >> 16));
                        const uint32_t dst = dst_base + (c8 >> 3) * L::kBox + rr * 128 + (((c8 & 7) ^ (rr & 7)) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w0), "r"(w1),
                                     "r"(w2), "r"(w3) : "memory");
                    }
                    fence_proxy_async_smem();             // the tensor core reads the copy through the async proxy
                    mbar_arrive(smem_u32(&bar_vf[sv]));
                    mbar_arrive(smem_u32(&bar_v8e[s8]));
                }
                if (!ok) break;
            }
            // ---- epilogue of the item
            const int par = it_n & 1;
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_stats[par]), (it_n >> 1) & 1, ctl, kBarStats))) break;
            const float m_a = xm[par][0][r_in_tile], m_b = xm[par][1][r_in_tile];
            const float m_fin = fmaxf(m_a, m_b);
            const float l_run = xsum[par][0][r_in_tile] * ex2_approx(m_a - m_fin) +
                                xsum[par][1][r_in_tile] * ex2_approx(m_b - m_fin);
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_stats_free[par]));
            float inv_l = 1.0f / l_run;
            if constexpr (FP8) inv_l *= v_scale[it.bh];
            const int row = it.q_start + r_in_tile;
            if (lse_out != nullptr && row < seq_len)
                lse_out[static_cast<size_t>(it.bh) * seq_len + row] = kLn2 * (m_fin + log2f(l_run));
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_odone), it_n & 1, ctl, kBarODone))) break;
            tc_fence_after();
            if constexpr (GQA) {
                // Result of this KV split for the rows that carry a (token, head) pair: with several
                // splits a normalised fp32 partial O and its LSE (the merge is a separate kernel), with
                // one split the final 16-bit O and the LSE.
                const bool live = r_in_tile < gq.live_rows && it.tok0 + r_in_tile / gq.group < gq.n_tok;
                const size_t pidx = gqa_partial_index(gq, it, r_in_tile);
                // a token with no visible key (a sequence shorter than the token count): O = 0, LSE = -inf
                const bool seen = l_run > 0.0f;
                if (!seen) inv_l = 0.0f;
                const bool direct = gq.n_splits == 1;     // nothing to merge: this is the result
                const float lse_val = seen ? kLn2 * (m_fin + log2f(l_run)) : -INFINITY;
                if (live) {
                    if (!direct) gq.lse_part[pidx] = lse_val;
                    else if (gq.lse_final != nullptr) gq.lse_final[pidx] = lse_val;
                }
#pragma unroll 1
                for (int c = 0; c < D / 32; c++) {
                    uint32_t o[32];
                    tmem_ld32_wait(t_o + c * 32, o);
                    if (c == D / 32 - 1) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&bar_ofree));
                    }
                    if (!seen) {                          // P was 2^(-inf + inf) there: not a number
#pragma unroll
                        for (int i = 0; i < 32; i++) o[i] = 0u;
                    }
                    if (live && direct) {
                        uint4* dst = reinterpret_cast<uint4*>(gq.o_final + pidx * D + c * 32);
#pragma unroll
                        for (int e = 0; e < 4; e++)
                            dst[e] = make_uint4(
                                pack_16<BF16>(__uint_as_float(o[8 * e]) * inv_l, __uint_as_float(o[8 * e + 1]) * inv_l),
                                pack_16<BF16>(__uint_as_float(o[8 * e + 2]) * inv_l, __uint_as_float(o[8 * e + 3]) * inv_l),
                                pack_16<BF16>(__uint_as_float(o[8 * e + 4]) * inv_l, __uint_as_float(o[8 * e + 5]) * inv_l),
                                pack_16<BF16>(__uint_as_float(o[8 * e + 6]) * inv_l, __uint_as_float(o[8 * e + 7]) * inv_l));
                    } else if (live) {
                        float4* dst = reinterpret_cast<float4*>(gq.o_part + pidx * D + c * 32);
#pragma unroll
                        for (int e = 0; e < 8; e++)
                            dst[e] = make_float4(__uint_as_float(o[4 * e]) * inv_l, __uint_as_float(o[4 * e + 1]) * inv_l,
                                                 __uint_as_float(o[4 * e + 2]) * inv_l, __uint_as_float(o[4 * e + 3]) * inv_l);
                    }
                }
                it_n++;
                continue;
            }
            // the staging buffer must have been drained by the previous item's TMA store
            if (tid == 384) tma_store_wait_read();
            if (!rendezvous4(0)) break;
#pragma unroll 1
            for (int c = 0; c < D / 32; c++) {
                uint32_t o[32];
                tmem_ld32_wait(t_o + c * 32, o);
                if (c == D / 32 - 1) {                    // the whole row is out of TMEM: the next item may overwrite O
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bar_ofree));
                }
#pragma unroll
                for (int g8 = 0; g8 < 4; g8++) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; e++)
                        w[e] = pack_16<BF16>(__uint_as_float(o[g8 * 8 + 2 * e]) * inv_l,
                                             __uint_as_float(o[g8 * 8 + 2 * e + 1]) * inv_l);
                    const int c16 = c * 4 + g8;           // 8-element (16-byte) group index in the row
                    const uint32_t addr = o_s + (c16 >> 3) * L::kBox + r_in_tile * 128 +
                                          (((c16 & 7) ^ (r_in_tile & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]),
                                 "r"(w[2]), "r"(w[3]) : "memory");
                }
            }
            fence_proxy_async_smem();
            if (!rendezvous4(1)) break;
            if (tid == 384) {
                for (int bx = 0; bx < NBOX; bx++)
                    tma_store_3d(&tm_o, o_s + bx * L::kBox, bx * 64, it.q_start, it.bh);
                tma_store_commit();
            }
            it_n++;
        }
        if (tid == 384) tma_store_wait_read();            // the CTA may exit once staging has been read
        __syncwarp();
    } else {
        // ------------------------------------------------------------ softmax + epilogue (warps 0-7)
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
        const int grp = warp >> 2;                        // group 0 owns even tiles (S0, P0), group 1 odd ones
        const int r_in_tile = (warp & 3) * 32 + lane;     // 0..127 == TMEM lane; one thread owns the whole row
        const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t t_o = tmem + lane_off + O_COL;
        int g0 = 0, it_n = 0;
        bool ok = true;

        for (int r = 0; ok && r < n_rounds; r++) {
            Item it;
            if (!get_item<CAUSAL, GQA, GROUPED>(r, n_items, n_bh, n_qtiles, seq_len, gq, it)) continue;
            const int row = it.q_start + r_in_tile;
            // keys [0,row_limit) visible.  Decode with several query tokens: they are the last n_tok
            // entries of the cache, token t sees everything up to and including itself.
            const int row_limit = CAUSAL ? min(seq_len, row + 1)
                                  : GQA  ? max(0, min(it.kv_len, it.kv_len - gq.n_tok + 1 + it.tok0 + r_in_tile / gq.group))
                                         : it.kv_len;
            const int tile_min_limit = CAUSAL ? min(seq_len, it.q_start + 1)
                                       : GQA  ? max(0, min(it.kv_len, it.kv_len - gq.n_tok + 1 + it.tok0)) : it.kv_len;
            float scale_log2 = scale_log2_in;
            if constexpr (FP8) scale_log2 *= q_scale[it.bh] * k_scale[it.bh];
            const uint64_t scale2 = pack2(scale_log2, scale_log2);
            // Running state of THIS thread: the reference max its partial row sum is expressed in.
            // The row's two threads alternate tiles; the max in use travels from tile to tile
            // through the tagged m_slot entries, so every tile of a row is exponentiated against
            // one agreed sequence.
            float m_mine = -1e30f;
            uint64_t lsum2 = pack2(0.0f, 0.0f);

            for (int j = (g0 & 1) == grp ? 0 : 1; j < it.n_kv; j += 2) {
                const int g = g0 + j;                     // global tile index; g & 1 == grp
                const int kv_start = (GQA ? it.t0 + j : j) * kBN;
                // The votes keep the warp together: every lane leaves the loop or none does.
                if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_qk[g % kRing]), (g / kRing) & 1, ctl, kBarSFull))) { ok = false; break; }
                tc_fence_after();
                const int u = g % kNU;                    // the tile's score buffer; P goes back into its first half
                const uint32_t t_s = tmem + lane_off + u * 128;
                if constexpr (GQA) {
                    // Decode: only the first `group` rows of the tile carry a query head.  A warp whose 32
                    // rows are all padding has nothing to compute: it keeps step with the tile (the wait
                    // above) and reports its part of P as done; whatever P V makes of those rows stays in
                    // rows that are never stored.
                    if ((warp & 3) * 32 >= gq.live_rows) {
                        tc_fence_before();
                        if (lane == 0) mbar_arrive(smem_u32(&bar_pf[u]));
                        continue;
                    }
                }
                uint32_t s[128];
                tmem_ld128_wait(t_s, s);
                if ((tile_min_limit - kv_start) < kBN) { // tile touches the mask or the ragged end
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
                // ---- the max in use: taken over from the previous tile (owned by the other group)
                // unless this tile's max exceeds it by more than the threshold
                float m_new = tile_max, m_prev_keep = tile_max;
                bool changed = false;
                const uint32_t slot = smem_u32(&m_slot[it_n & 1][r_in_tile]);
                if (j > 0) {
                    // poll for the previous tile's entry (normally long there); bounded like every wait
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
                            atomicCAS(ctl.status, 0, wait_timeout_word(kBarM));
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
                if (m_new != m_mine) {                    // bring this thread's partial sum to the new reference
                    const float f = ex2_approx(m_mine - m_new);
                    lsum2 = fma2(lsum2, pack2(f, f), pack2(0.0f, 0.0f));
                }

                // ---- rare: the max in use grew -> rescale O in TMEM before this tile's P V
                if (__any_sync(0xffffffffu, changed)) {
                    // P V(g-1) must have finished accumulating into O
                    if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_pvd[(g - 1) % kRing]), ((g - 1) / kRing) & 1, ctl, kBarPV))) { ok = false; break; }
                    tc_fence_after();
                    // rows whose max did not change multiply by one; m_mine is not the previous max of
                    // the ROW (the other thread may have moved it), so the factor comes from m_prev
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

                // ---- p = 2^(s*scale*log2e - m); row sum; P -> TMEM as packed 16-bit pairs, over the
                // first 64 columns of the scores they came from (this thread's own lane, already in
                // registers), so the softmax never waits for a P buffer: the next tile's exponentials
                // do not depend on this tile's P V
                const uint64_t negm2 = pack2(-m_new, -m_new);
                uint64_t acc0 = lsum2, acc1 = pack2(0.0f, 0.0f), acc2 = acc1, acc3 = acc1;   // independent sum chains
                constexpr int NCHUNK = 4;                 // P is stored 32 columns at a time
                constexpr int PAIRS = 64 / NCHUNK;        // 16-bit pairs (TMEM columns of P) per store
#pragma unroll
                for (int c = 0; c < NCHUNK; c++) {
                    uint32_t pk[PAIRS];
#pragma unroll
                    for (int i = 0; i < PAIRS; i++) {
                        const int e = 2 * (c * PAIRS + i);
                        const uint64_t t = fma2(pack2(__uint_as_float(s[e]), __uint_as_float(s[e + 1])), scale2, negm2);
                        float t0, t1;
                        unpack2(t, t0, t1);
                        const float p0 = ex2_approx(t0), p1 = ex2_approx(t1);
                        const uint64_t pp = pack2(p0, p1);
                        if ((i & 3) == 0) acc0 = add2(acc0, pp);
                        else if ((i & 3) == 1) acc1 = add2(acc1, pp);
                        else if ((i & 3) == 2) acc2 = add2(acc2, pp);
                        else acc3 = add2(acc3, pp);
                        pk[i] = pack_16<P_BF16>(p0, p1);
                    }
#pragma unroll
                    for (int q = 0; q < PAIRS / 16; q++)
                        tmem_st_x16(t_s + c * PAIRS + q * 16, *reinterpret_cast<uint32_t (*)[16]>(&pk[q * 16]));
                }
                lsum2 = add2(add2(acc0, acc1), add2(acc2, acc3));
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar_pf[u]));
            }
            if (!ok) break;

            {
                // ---- end of the item: hand (reference max, partial row sum) to the epilogue warps and
                // go straight on to the next item
                const int par = it_n & 1;
                if (it_n >= 2 &&
                    !__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_stats_free[par]), ((it_n >> 1) - 1) & 1, ctl, kBarStatsFree))) { ok = false; break; }
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

    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem, TMEM_COLS);
}

// How many heads the work list walks at a time: as many as keep their K and V (which every query
// tile of a head re-reads) inside a share of L2.  Measured on 32 heads of S=8192, d_head 128
// (134 MB of K and V against 126 MB of L2): walking all heads at once streams K/V from HBM.
constexpr long long kGroupBytes = FA_GROUP_MB * 1024ll * 1024ll;
constexpr long long kNoGroupBytes = 64ll * 1024 * 1024;      // half of L2
int heads_per_group(int n_bh, int seq_len, int d_head, int elem_bytes) {
    const long long per_head = 2ll * seq_len * d_head * elem_bytes;
    if (per_head * n_bh <= kNoGroupBytes) return n_bh;        // all of K and V fits comfortably: one group
    long long g = kGroupBytes / (per_head > 0 ? per_head : 1);
    if (g < 1) g = 1;
    if (g > n_bh) g = n_bh;
    return (int)g;
}

template <int D, bool CAUSAL, bool BF16, bool FP8>
int launch_instance(const fa_prefill_args& a, DeviceState* st, const CUtensorMap& tq,
                    const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to) {
    using L = PrefillSmem<D, FP8, false>;
    const int n_bh = a.batch_size * a.num_heads;
    GqaDev order{};
    order.group = heads_per_group(n_bh, a.seq_len, a.d_head, FP8 ? 1 : 2);
    const bool grouped = order.group < n_bh;
    auto kernel = grouped ? prefill_kernel<D, CAUSAL, BF16, FP8, false, true>
                          : prefill_kernel<D, CAUSAL, BF16, FP8, false, false>;
    static bool configured[64][2] = {};
    if (!configured[st->device][grouped]) {
        FA_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
        configured[st->device][grouped] = true;
    }
    const int n_qtiles = (a.seq_len + kBM - 1) / kBM;
    const long long n_items = (long long)n_bh * n_qtiles;
    if (n_items > 0x7FFFFFFFll) return FA_ERR_INVALID_ARGUMENT;
    const unsigned grid = (unsigned)(n_items < st->sm_count ? n_items : st->sm_count);
    kernel<<<grid, kThreads, L::kTotal, static_cast<cudaStream_t>(a.stream)>>>(
        tq, tk, tv, to, a.lse, a.seq_len, n_bh, n_qtiles, (int)n_items, a.scale * kLog2e, a.q_scale,
        a.k_scale, a.v_scale, st->status, order);
    FA_CUDA_TRY(cudaGetLastError());
    return FA_OK;
}

template <int D, bool BF16, bool FP8>
int launch_gqa_instance(const GqaLaunch& g, DeviceState* st, const CUtensorMap& tq, const CUtensorMap& tk,
                        const CUtensorMap& tv) {
    using L = PrefillSmem<D, FP8>;
    auto kernel = prefill_kernel<D, false, BF16, FP8, true, false>;
    static bool configured[64] = {};
    if (!configured[st->device]) {
        FA_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
        configured[st->device] = true;
    }
    const int n_bh = g.batch * g.n_kv_heads;
    const int tok_per_tile = kBM / g.group < g.n_tok ? kBM / g.group : g.n_tok;
    const int n_qt = (g.n_tok + tok_per_tile - 1) / tok_per_tile;
    const long long n_items = (long long)n_bh * n_qt * g.n_splits;
    if (n_items > 0x7FFFFFFFll) return FA_ERR_INVALID_ARGUMENT;
    const unsigned grid = (unsigned)(n_items < st->sm_count ? n_items : st->sm_count);
    int page_shift = 0;
    while ((1 << page_shift) < g.page_size) page_shift++;
    const GqaDev gq{g.o_part, g.lse_part, static_cast<uint16_t*>(g.o_final), g.lse_final, g.n_splits,
                    g.tiles_per_split, g.group, g.n_kv_heads,
                    g.n_tok, tok_per_tile, n_qt, tok_per_tile * g.group, g.seq_lens, g.block_table, g.table_stride,
                    page_shift};
    kernel<<<grid, kThreads, L::kTotal, g.stream>>>(tq, tk, tv, tq, nullptr, g.kv_len, n_bh, 1, (int)n_items,
                                                    g.scale * kLog2e, g.q_scale, g.k_scale, g.v_scale, st->status, gq);
    FA_CUDA_TRY(cudaGetLastError());
    return FA_OK;
}

}  // namespace

// Which of the two prefill kernels runs a problem (the reference's dispatcher picks its tile
// variant by the same kind of rule, kernels/flash_attention.cu:595-617).  The kernel with two
// query tiles per CTA needs the pairs alone to fill the GPU; below that the one-tile kernel
// spreads a small problem over twice as many SMs and has the shorter critical path.
std::atomic<int> g_prefill_variant{FA_PREFILL_AUTO};

int choose_prefill_variant(int batch_size, int num_heads, int seq_len, int d_head, const DeviceState* st) {
    const int v = g_prefill_variant.load(std::memory_order_relaxed);
    if (v != FA_PREFILL_AUTO) return v;
    (void)batch_size; (void)num_heads; (void)seq_len; (void)d_head; (void)st;
    return FA_PREFILL_ONE_TILE;
}

int launch_prefill_16bit(const fa_prefill_args& a, DeviceState* st, int variant) {
    const uint64_t n_bh = (uint64_t)a.batch_size * a.num_heads;
    CUtensorMap tq, tk, tv, to;
    int rc;
    if ((rc = make_tensor_map_3d(&tq, a.q, a.dtype, a.d_head, a.seq_len, n_bh, 64, kBM)) != FA_OK) return rc;
    if ((rc = make_tensor_map_3d(&tk, a.k, a.dtype, a.d_head, a.seq_len, n_bh, 64, kBN)) != FA_OK) return rc;
    if ((rc = make_tensor_map_3d(&tv, a.v, a.dtype, a.d_head, a.seq_len, n_bh, 64, kBN)) != FA_OK) return rc;
    if ((rc = make_tensor_map_3d(&to, a.o, a.dtype, a.d_head, a.seq_len, n_bh, 64, kBM)) != FA_OK) return rc;
    if (variant == FA_PREFILL_AUTO) variant = choose_prefill_variant(a.batch_size, a.num_heads, a.seq_len, a.d_head, st);
    if (variant == FA_PREFILL_CTA_PAIR && a.d_head == 128)     // built for d_head 128 only; d_head 64 takes the one-tile kernel
        return launch_prefill_2sm_16bit(a, st, heads_per_group((int)n_bh, a.seq_len, a.d_head, 2));
    if (variant == FA_PREFILL_TILE_PAIR) return launch_prefill_pair_16bit(a, st, heads_per_group((int)n_bh, a.seq_len, a.d_head, 2), tq, tk, tv, to);
    const bool bf = a.dtype == FA_DTYPE_BF16;
    const bool causal = a.causal != 0;
#define FA_DISPATCH(DH)                                                                      \
    (causal ? (bf ? launch_instance<DH, true, true, false>(a, st, tq, tk, tv, to)            \
                  : launch_instance<DH, true, false, false>(a, st, tq, tk, tv, to))          \
            : (bf ? launch_instance<DH, false, true, false>(a, st, tq, tk, tv, to)           \
                  : launch_instance<DH, false, false, false>(a, st, tq, tk, tv, to)))
    if (a.d_head == 64) return FA_DISPATCH(64);
    return FA_DISPATCH(128);
#undef FA_DISPATCH
}

int launch_decode_gqa(const GqaLaunch& g, DeviceState* st) {
    CUtensorMap tq, tk, tv;
    int rc;
    // Q [B, T, Hq, D]: one box per (batch, KV head) with its group x T rows, token-major
    const bool e4m3 = g.dtype == FA_DTYPE_E4M3;
    const uint32_t box_cols = e4m3 ? 128 : 64;           // 128 bytes of a row either way
    if ((rc = make_tensor_map_q5(&tq, g.q, g.dtype, g.d_head, g.group, g.n_tok, g.n_kv_heads, g.batch, box_cols)) != FA_OK)
        return rc;
    // dense / strided cache: (d, key, KV head, batch); paged: (d, key in page, KV head, page)
    const bool paged = g.block_table != nullptr;
    const uint64_t rows = paged ? (uint64_t)g.page_size : (uint64_t)g.kv_len;
    const uint64_t blocks = paged ? (uint64_t)g.n_pages : (uint64_t)g.batch;
    const uint64_t bstride = paged ? (uint64_t)g.page_stride : (uint64_t)g.batch_stride;
    const uint32_t box_rows = paged && g.page_size < kBN ? (uint32_t)g.page_size : (uint32_t)kBN;
    if ((rc = make_tensor_map_4d(&tk, g.k, g.dtype, g.d_head, rows, g.n_kv_heads, blocks, g.row_stride,
                                 g.head_stride, bstride, box_cols, box_rows)) != FA_OK) return rc;
    if ((rc = make_tensor_map_4d(&tv, g.v, g.dtype, g.d_head, rows, g.n_kv_heads, blocks, g.row_stride,
                                 g.head_stride, bstride, box_cols, box_rows)) != FA_OK) return rc;
    if (e4m3) return launch_gqa_instance<128, true, true>(g, st, tq, tk, tv);
    const bool bf = g.dtype == FA_DTYPE_BF16;
    if (g.d_head == 64)
        return bf ? launch_gqa_instance<64, true, false>(g, st, tq, tk, tv) : launch_gqa_instance<64, false, false>(g, st, tq, tk, tv);
    return bf ? launch_gqa_instance<128, true, false>(g, st, tq, tk, tv) : launch_gqa_instance<128, false, false>(g, st, tq, tk, tv);
}


// e4m3 codes -> fp16 (exact), 16 codes per thread.
__global__ void e4m3_to_f16_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long n16) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n16) return;
    const uint4 c = src[i];
    const uint32_t w[4] = {c.x, c.y, c.z, c.w};
    uint4 lo, hi;
    lo.x = e4m3x2_to_f16x2(static_cast<uint16_t>(w[0] & 0xFFFFu)); lo.y = e4m3x2_to_f16x2(static_cast<uint16_t>(w[0] >> 16));
    lo.z = e4m3x2_to_f16x2(static_cast<uint16_t>(w[1] & 0xFFFFu)); lo.w = e4m3x2_to_f16x2(static_cast<uint16_t>(w[1] >> 16));
    hi.x = e4m3x2_to_f16x2(static_cast<uint16_t>(w[2] & 0xFFFFu)); hi.y = e4m3x2_to_f16x2(static_cast<uint16_t>(w[2] >> 16));
    hi.z = e4m3x2_to_f16x2(static_cast<uint16_t>(w[3] & 0xFFFFu)); hi.w = e4m3x2_to_f16x2(static_cast<uint16_t>(w[3] >> 16));
    dst[2 * i] = lo;
    dst[2 * i + 1] = hi;
}

// e4m3 inputs (d_head 128), bf16 output.  V is converted to fp16 once, into a stream-ordered
// scratch allocation (cudaMallocFromPoolAsync / cudaFreeAsync on the caller's stream) that lives
// for the call (converting every V tile in shared memory inside the
// kernel made this path slower than bf16: 0.57 against 0.44 ms on B=8 H=16 S=4096 causal); heads
// are taken in chunks so that the scratch stays below kFp8ScratchBytes.
constexpr size_t kFp8ScratchBytes = 256ull << 20;
int launch_prefill_fp8(const fa_prefill_args& a, DeviceState* st) {
    const uint64_t n_bh = (uint64_t)a.batch_size * a.num_heads;
    const size_t head_elems = (size_t)a.seq_len * 128;             // per head and tensor
    uint64_t chunk = kFp8ScratchBytes / (head_elems * 2);
    if (chunk < 1) chunk = 1;
    if (chunk > n_bh) chunk = n_bh;
    cudaStream_t stream = static_cast<cudaStream_t>(a.stream);
    // The scratch comes from a pool of the library's own whose release threshold is unlimited: the
    // process's default pool would hand the memory back at every synchronisation and the next call
    // would pay for a fresh allocation (measured: 4 ms on the first call after a synchronise).
    if (!st->pool_ready.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(st->pool_mutex);
        if (!st->pool_ready.load(std::memory_order_relaxed)) {
            cudaMemPoolProps props = {};
            props.allocType = cudaMemAllocationTypePinned;
            props.handleTypes = cudaMemHandleTypeNone;
            props.location.type = cudaMemLocationTypeDevice;
            props.location.id = st->device;
            FA_CUDA_TRY(cudaMemPoolCreate(&st->scratch_pool, &props));
            uint64_t keep = UINT64_MAX;
            FA_CUDA_TRY(cudaMemPoolSetAttribute(st->scratch_pool, cudaMemPoolAttrReleaseThreshold, &keep));
            st->pool_ready.store(true, std::memory_order_release);
        }
    }
    void* v16 = nullptr;
    FA_CUDA_TRY(cudaMallocFromPoolAsync(&v16, chunk * head_elems * 2, st->scratch_pool, stream));
    int rc = FA_OK;
    for (uint64_t h0 = 0; h0 < n_bh && rc == FA_OK; h0 += chunk) {
        const uint64_t nh = (n_bh - h0 < chunk) ? n_bh - h0 : chunk;
        // this chunk's heads as a problem of its own: batch 1 x nh heads
        fa_prefill_args c = a;
        c.batch_size = 1;
        c.num_heads = (int)nh;
        c.q = static_cast<const uint8_t*>(a.q) + h0 * head_elems;
        c.k = static_cast<const uint8_t*>(a.k) + h0 * head_elems;
        c.v = static_cast<const uint8_t*>(a.v) + h0 * head_elems;
        c.o = static_cast<uint16_t*>(a.o) + h0 * head_elems;
        if (a.lse) c.lse = a.lse + h0 * a.seq_len;
        c.q_scale = a.q_scale + h0;
        c.k_scale = a.k_scale + h0;
        c.v_scale = a.v_scale + h0;
        const long long n16 = (long long)(nh * head_elems / 16);
        e4m3_to_f16_kernel<<<(unsigned)((n16 + 255) / 256), 256, 0, stream>>>(static_cast<const uint4*>(c.v),
                                                                            static_cast<uint4*>(v16), n16);
        if (cudaGetLastError() != cudaSuccess) { rc = FA_ERR_CUDA; break; }
        CUtensorMap tq, tk, tv, to;
        if ((rc = make_tensor_map_3d(&tq, c.q, FA_DTYPE_E4M3, 128, a.seq_len, nh, 128, kBM)) != FA_OK) break;
        if ((rc = make_tensor_map_3d(&tk, c.k, FA_DTYPE_E4M3, 128, a.seq_len, nh, 128, kBN)) != FA_OK) break;
        if ((rc = make_tensor_map_3d(&tv, v16, FA_DTYPE_F16, 128, a.seq_len, nh, 64, kBN)) != FA_OK) break;
        if ((rc = make_tensor_map_3d(&to, c.o, FA_DTYPE_BF16, 128, a.seq_len, nh, 64, kBM)) != FA_OK) break;
        rc = a.causal ? launch_instance<128, true, true, true>(c, st, tq, tk, tv, to)
                      : launch_instance<128, false, true, true>(c, st, tq, tk, tv, to);
    }
    const cudaError_t fe = cudaFreeAsync(v16, stream);            // after the last kernel that reads it, in stream order
    if (rc == FA_OK && fe != cudaSuccess) rc = FA_ERR_CUDA;
    return rc;
}

}  // namespace fa
