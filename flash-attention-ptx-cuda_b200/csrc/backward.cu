// Backward pass of the attention forward in prefill.cu: dQ, dK, dV from dO and
// the log-sum-exp the forward saved.
//
// The reference has no backward; its forward kernel stores L "for the backward
// pass" (kernels/flash_attention.cu:497).  The mathematics is that of its
// forward (src/demo.cu:28-70) differentiated:
//     P  = exp(S * scale - LSE),  S = Q K^T          (masked entries: P = 0)
//     dV = P^T dO
//     dP = dO V^T
//     dS = P o (dP - delta) * scale,  delta_i = sum_d dO_id O_id
//     dQ = dS K,   dK = dS^T Q
//
// Three kernels, no atomics:
//   delta_kernel          delta = rowsum(dO o O), fp32.
//   bwd_kernel<MODE 0>    dK and dV.  A work item is one key tile of one head: its K and V
//                         tiles stay in shared memory, the query tiles stream past; per step
//                         S^T = K Q^T and dP^T = V dO^T on the tensor core (so a thread owns
//                         a KEY row in TMEM), P^T and dS^T go back to TMEM as 16-bit, then
//                         dV += P^T dO and dK += dS^T Q with those as the TMEM operand.
//   bwd_kernel<MODE 1>    dQ.  A work item is one query tile of one head: Q and dO stay, the
//                         key tiles stream; S = Q K^T, dP = dO V^T, dS to TMEM, dQ += dS K.
//                         (S and dP are computed twice overall; nothing is accumulated
//                         across CTAs.)
// Both modes are the same code: two stationary tiles A0, A1, two streamed tiles B0, B1 per
// step, products T0 = A0 B0^T and T1 = A1 B1^T, accumulators fed from TMEM.  The CTAs are
// persistent (one per SM, a static work list each): TMEM and barriers are set up once, and
// the loads and products of an item's first steps overlap the last steps and the output of
// the item before.
// A step streams 64 rows.  Even steps (counted over the CTA's whole work list) use one TMEM
// product buffer, odd steps the other, and each parity has its own compute warps and its own
// product issuer, so the two chains
//     products(t) -> exponentials, dS -> accumulating MMAs(t)
// run a step apart and fill each other's waits.  The 16-bit operands of the accumulating
// MMAs get TMEM columns of their own, so a product buffer is free again as soon as its
// values are in registers (d_head 128, MODE 0 has no columns left for that: there the
// operands overwrite the products and the buffer is free when the accumulations are done).
//   warps 0-7    even steps, two threads per stationary row (TMEM lane): warps 0-3 take the
//                first 32 streamed columns of a step, warps 4-7 the other 32: exponentials,
//                dS, 16-bit operands to TMEM; at the end of an item conversion of the
//                accumulators.
//   warps 8-15   the same for odd steps.
//   warps 16, 17 lane 0 issues the product MMAs of even / odd steps.
//   warps 18, 19 lane 0 issues the accumulating MMAs, one accumulator each (dV and dK; the
//                dQ kernel uses warp 18 only), every step in order.
//   warp 20      lane 0 issues the TMA loads: stationary tiles (two buffers at d_head 64, so
//                the next item's arrive early) and the streamed stages.
//   warp 21      allocates TMEM; at d_head 64 it also issues the TMA stores of the output
//                tiles, which the compute warps stage in the stationary buffer the finished
//                item no longer needs (row-strided stores straight from registers cost an L2
//                write transaction per 16 or 32 bytes and took 1300-2800 clocks per item).
// An MMA costs its issuing thread 55-110 clocks whatever its size, and two threads issue twice
// as many (measured), so every MMA stream has a thread of its own; and the per-step waits of
// a compute warp (products ready, operand columns free, stores complete) are latencies that
// only other warps' work can fill, hence sixteen compute warps on two steps rather than
// eight on one.
#include <cmath>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_common.h"
#include "ptx.cuh"
#include "tmem_ld.cuh"

namespace fa {
namespace {

constexpr int kT = 128;                  // tile edge: stationary rows per CTA
constexpr int kBwdThreads = 768;         // 24 warps (22, 23 idle: register pools move by groups of four warps)
constexpr int kComputeWarps = 16;
constexpr int kProdWarp = 16;            // 16, 17: product MMAs of even / odd steps
constexpr int kAccWarp = 18;             // 18, 19: accumulating MMAs, one accumulator each
constexpr int kLoadWarp = 20;            // TMA loads
constexpr int kTmemWarp = 21;            // TMEM allocation and release; TMA stores of staged output tiles
constexpr int kW = 64;                   // streamed rows per step (columns of one product)
constexpr float kLog2e = 1.4426950408889634f;
// setmaxnreg moves registers inside the pool the CTA got at launch (threads x registers at launch)
constexpr int kBwdRegsLaunch = (65536 / kBwdThreads) / 8 * 8;
constexpr int kBwdRegsCompute = 104;     // warps 0-15
constexpr int kBwdRegsRest = 32;         // warps 16-23
static_assert(512 * kBwdRegsCompute + 256 * kBwdRegsRest <= kBwdThreads * kBwdRegsLaunch,
              "setmaxnreg targets exceed the CTA's register pool");

enum : int { kBwdBarA = 21, kBwdBarFull = 22, kBwdBarT = 23, kBwdBarP = 24, kBwdBarFree = 25, kBwdBarDone = 26, kBwdBarAcc = 27 };

template <int D>
struct BwdSmem {
    static constexpr int kNBox = D / 64;              // 64-column (128-byte) boxes per row
    static constexpr int kBox = 128 * 128;            // one box: 128 rows x 128 bytes
    static constexpr int kTile = kNBox * kBox;        // one 128 x D 16-bit tile (stationary operands)
    static constexpr int kBoxB = kW * 128;            // one box of a streamed tile: kW rows x 128 bytes
    static constexpr int kTileB = kNBox * kBoxB;      // one kW x D streamed tile
    // streamed (B0, B1) tile pairs in flight: a pair is requested when the accumulations of the
    // step that held its stage have completed, and a load takes longer than a step
    static constexpr int kStages = (D == 64) ? 8 : 4;
    // buffers of the stationary tile pair: with two, an item's tiles arrive while the item before
    // still computes (d_head 128 has no room for a second pair)
    static constexpr int kNA = (D == 64) ? 2 : 1;
    static constexpr int kTotal = kNA * 2 * kTile + kStages * 2 * kTileB + 1024;
};

// TMEM column, relative to the operand's first, of the 16-bit slice for streamed rows
// [16 kk, 16 kk + 16) of a step.  Each half of a parity's compute warps writes 16 columns of pairs:
// side by side where the operands have columns of their own; in place each half writes over the
// start of the 32 fp32 columns it has read, so the slices of streamed rows 32-63 start at column 32.
__host__ __device__ constexpr uint32_t op16_col(int kk, bool in_place) {
    return in_place ? (kk < 2 ? 0u : 32u) + (kk & 1) * 8u : kk * 8u;
}

// delta = rowsum(dO o O).  d_head / 8 lanes per row, 16 bytes of each tensor per lane: a warp
// covers 4 rows (d_head 64) or 2 (d_head 128) with one load instruction per tensor.
template <bool BF16>
__global__ void delta_kernel(const uint16_t* __restrict__ o, const uint16_t* __restrict__ d_o,
                             float* __restrict__ delta, long long n_rows, int d_head) {
    const int lanes_per_row = d_head >> 3;                       // 8 or 16
    const int rows_per_warp = 32 / lanes_per_row;
    const int lane = threadIdx.x & 31;
    const long long warp_id = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long row = warp_id * rows_per_warp + lane / lanes_per_row;
    const int c = (lane % lanes_per_row) * 8;
    float acc = 0.0f;
    if (row < n_rows) {
        const uint4 a = *reinterpret_cast<const uint4*>(o + row * d_head + c);
        const uint4 b = *reinterpret_cast<const uint4*>(d_o + row * d_head + c);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float a0, a1, b0, b1;
            if constexpr (BF16) {
                a0 = __uint_as_float(aw[i] << 16); a1 = __uint_as_float(aw[i] & 0xFFFF0000u);
                b0 = __uint_as_float(bw[i] << 16); b1 = __uint_as_float(bw[i] & 0xFFFF0000u);
            } else {
                const float2 fa2 = __half22float2(*reinterpret_cast<const __half2*>(&aw[i]));
                const float2 fb2 = __half22float2(*reinterpret_cast<const __half2*>(&bw[i]));
                a0 = fa2.x; a1 = fa2.y; b0 = fb2.x; b1 = fb2.y;
            }
            acc = fmaf(a0, b0, fmaf(a1, b1, acc));
        }
    }
    for (int off = lanes_per_row >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (row < n_rows && (lane % lanes_per_row) == 0) delta[row] = acc;
}

// One unit of work: one stationary tile of one head and the rows that stream past it.
struct BwdItem {
    int bh, tile;
    int row0;        // first streamed row
    int n_steps;     // steps of kW streamed rows
};

// Work list of a CTA: items round * gridDim.x + (this CTA's place in the round), the place running
// forwards in even rounds and backwards in odd ones so that the per-CTA totals even out.  Under the
// causal mask the heaviest tiles of every head come first (key tile 0 / the last query tile have the
// most steps); without it the tiles of a head stay together so that its streamed rows stay in L2.
template <bool CAUSAL, int MODE>
__device__ __forceinline__ bool bwd_item(int round, int n_items, int n_bh, int n_tiles, int seq_len, BwdItem& it) {
    const int G = gridDim.x, c = blockIdx.x;
    const int idx = (round & 1) ? round * G + (G - 1 - c) : round * G + c;
    if (idx >= n_items) return false;
    int slot_x;
    if (CAUSAL) { slot_x = idx / n_bh; it.bh = idx - slot_x * n_bh; }
    else        { it.bh = idx / n_tiles; slot_x = idx - it.bh * n_tiles; }
    it.tile = (MODE == 0) ? slot_x : (n_tiles - 1 - slot_x);
    it.row0 = (MODE == 0 && CAUSAL) ? it.tile * kT : 0;
    const int row_end = (MODE == 1 && CAUSAL) ? min(seq_len, (it.tile + 1) * kT) : seq_len;
    it.n_steps = (row_end - it.row0 + kW - 1) / kW;
    return true;
}

// MODE 0: dK and dV of key tiles.  MODE 1: dQ of query tiles.  Persistent: one CTA per SM walks
// its work list, so that TMEM allocation and barrier set-up are paid once and the loads and
// products of an item's first steps overlap the last steps and the output of the item before.
// ta0 / ta1: maps of the stationary tensors (boxes of 128 rows); tb0 / tb1: maps of the streamed
// tensors (boxes of kW rows).
template <int D, bool CAUSAL, bool BF16, int MODE>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_kernel(const __grid_constant__ CUtensorMap ta0, const __grid_constant__ CUtensorMap ta1,
           const __grid_constant__ CUtensorMap tb0, const __grid_constant__ CUtensorMap tb1,
           const __grid_constant__ CUtensorMap to0, const __grid_constant__ CUtensorMap to1,
           const float* __restrict__ lse, const float* __restrict__ delta, uint16_t* __restrict__ out0,
           uint16_t* __restrict__ out1, int seq_len, int n_tiles, int n_bh, int n_items, float scale, int* status) {
    using L = BwdSmem<D>;
    constexpr int NBOX = L::kNBox, kStages = L::kStages, NA = L::kNA;
    constexpr uint32_t FMT = BF16 ? kFmtBF16 : kFmtF16;
    constexpr int NACC = (MODE == 0) ? 2 : 1;             // accumulators = accumulation issuers
    // TMEM: two product buffers of 128 columns (T0 in the first kW, T1 in the second kW), the
    // accumulators, then the 16-bit operands of each parity (P^T in 32 columns, dS in the next 32).
    // d_head 128, MODE 0: the accumulators take what is left, the operands overwrite the start of
    // T0 / T1.
    constexpr bool INPLACE = (MODE == 0 && D == 128);
    constexpr uint32_t ACC0_COL = 256, ACC1_COL = 256 + D;
    constexpr uint32_t OP_COL = 256 + NACC * D;
    static_assert(ACC1_COL + (MODE == 0 ? D : 0) <= 512 && (INPLACE || OP_COL + 128 <= 512), "TMEM columns");
    constexpr uint32_t OPP0 = INPLACE ? 0u : OP_COL, OPD0 = INPLACE ? (uint32_t)kW : OP_COL + 32;   // parity 0
    constexpr uint32_t OP_STRIDE = INPLACE ? 128u : 64u;                                             // to parity 1
    // With two stationary buffers the one an item has finished with is idle until the item after
    // next: the accumulators are staged there as 16-bit tiles and leave by TMA store while the next
    // item runs.  With one buffer the threads store their rows themselves.
    constexpr bool STAGED = (NA == 2);

    extern __shared__ uint8_t smem_raw[];
    // Every barrier completes one phase per use, uses counted over the CTA's whole work list:
    //   bar_a[b] / bar_afree[b]   stationary tiles of buffer b loaded / no longer read by any product
    //   bar_full[s] / bar_acc[s]  streamed tiles of stage s loaded / the accumulations that read them done
    //   bar_t[g] / bar_tfree[g]   products of parity g done / their values are in registers
    //   bar_p[g]                  16-bit operands of parity g in TMEM
    //   bar_done / bar_accfree    an item's accumulators complete / read out
    //   bar_ostaged / bar_ofree[b] an item's output tiles staged in buffer b / read by their TMA store
    __shared__ __align__(8) uint64_t bar_a[2], bar_afree[2], bar_full[kStages], bar_acc[kStages], bar_t[2], bar_tfree[2],
        bar_p[2], bar_done, bar_accfree, bar_ostaged, bar_ofree[2];
    // MODE 0: statistics of the streamed queries of the current / next step, per column pair
    // {-lse*log2e (col 0, col 1), -delta*scale (col 0, col 1)}: the addends of the two packed FMAs.
    // WARP_STATS: every compute warp stages the 32 columns it works on itself (lane j: column j), so
    // a __syncwarp orders writes and reads and the warps of a parity need not meet.  Otherwise
    // (d_head 128, where that measured 9 % slower) threads 0..63 of a parity stage its 64 columns
    // and the parity's eight warps meet at a named barrier once per step.
    constexpr bool WARP_STATS = !INPLACE;
    __shared__ __align__(16) float st_neg[MODE != 0 ? 1 : (WARP_STATS ? kComputeWarps : 2)][2][WARP_STATS ? 16 : 32][4];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t b_s = base + NA * 2 * L::kTile;        // stationary buffers first, then the stages
    WaitCtl ctl{&abort_flag, status};

    if (MODE == 0 && tid == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (tid == 0) {
        for (int i = 0; i < 2; i++) { mbar_init(smem_u32(&bar_a[i]), 1); mbar_init(smem_u32(&bar_afree[i]), 2); }
        for (int i = 0; i < kStages; i++) { mbar_init(smem_u32(&bar_full[i]), 1); mbar_init(smem_u32(&bar_acc[i]), NACC); }
        for (int i = 0; i < 2; i++) {
            mbar_init(smem_u32(&bar_t[i]), 1);
            mbar_init(smem_u32(&bar_tfree[i]), 8);       // one arrival per compute warp of the parity
            mbar_init(smem_u32(&bar_p[i]), 8);
        }
        mbar_init(smem_u32(&bar_done), NACC);
        mbar_init(smem_u32(&bar_accfree), kComputeWarps);
        mbar_init(smem_u32(&bar_ostaged), kComputeWarps);
        for (int i = 0; i < 2; i++) mbar_init(smem_u32(&bar_ofree[i]), 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == kTmemWarp) tmem_alloc(smem_u32(&tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    if (warp >= kComputeWarps) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kBwdRegsRest));

    // gs: steps of the items this CTA has finished; a step's place in every ring is gs + t
    if (warp == kLoadWarp) {
        // ------------------------------------------------------------ TMA loads (one thread)
        if (lane == 0) {
            BwdItem it;
            int gs = 0;
            bool ok = true;
            for (int k = 0; ok && bwd_item<CAUSAL, MODE>(k, n_items, n_bh, n_tiles, seq_len, it); k++) {
                const int buf = k % NA, use = k / NA;
                // the stationary tiles of item k - NA were last read by its products; where that item's
                // output was staged in the same buffer, by the TMA store of that output
                if (use >= 1 && !mbar_wait(smem_u32(STAGED ? &bar_ofree[buf] : &bar_afree[buf]), (use - 1) & 1, ctl, kBwdBarFree)) break;
                const uint32_t a0_s = base + buf * 2 * L::kTile, a1_s = a0_s + L::kTile;
                mbar_arrive_expect_tx(smem_u32(&bar_a[buf]), 2 * L::kTile);
                for (int b = 0; b < NBOX; b++) {
                    tma_load_3d(a0_s + b * L::kBox, &ta0, smem_u32(&bar_a[buf]), b * 64, it.tile * kT, it.bh);
                    tma_load_3d(a1_s + b * L::kBox, &ta1, smem_u32(&bar_a[buf]), b * 64, it.tile * kT, it.bh);
                }
                for (int t = 0; t < it.n_steps; t++) {
                    const int T = gs + t, s = T % kStages;
                    // the stage held step T - kStages: its accumulations must have completed
                    if (T >= kStages && !mbar_wait(smem_u32(&bar_acc[s]), ((T - kStages) / kStages) & 1, ctl, kBwdBarFree)) { ok = false; break; }
                    const uint32_t dst = b_s + s * 2 * L::kTileB;
                    mbar_arrive_expect_tx(smem_u32(&bar_full[s]), 2 * L::kTileB);
                    for (int b = 0; b < NBOX; b++) {
                        tma_load_3d(dst + b * L::kBoxB, &tb0, smem_u32(&bar_full[s]), b * 64, it.row0 + t * kW, it.bh);
                        tma_load_3d(dst + L::kTileB + b * L::kBoxB, &tb1, smem_u32(&bar_full[s]), b * 64, it.row0 + t * kW, it.bh);
                    }
                }
                gs += it.n_steps;
            }
        }
        __syncwarp();
    } else if (warp == kProdWarp || warp == kProdWarp + 1) {
        // ------------------------------------------------------------ product MMAs of one parity (one thread)
        if (lane == 0) {
            const int g = warp - kProdWarp;
            constexpr uint32_t idesc_t = make_idesc(kT, kW, FMT, FMT, kMajorK, kMajorK);
            constexpr uint64_t hi_k = make_sdesc_hi(16, 1024);
            const uint32_t tb = tmem + g * 128;
            BwdItem it;
            int gs = 0;
            bool ok = true;
            for (int k = 0; ok && bwd_item<CAUSAL, MODE>(k, n_items, n_bh, n_tiles, seq_len, it); k++) {
                const int buf = k % NA, use = k / NA;
                const uint32_t a0_s = base + buf * 2 * L::kTile, a1_s = a0_s + L::kTile;
                if (!mbar_wait(smem_u32(&bar_a[buf]), use & 1, ctl, kBwdBarA)) break;
                bool issued = false;
                for (int t = (g ^ gs) & 1; t < it.n_steps; t += 2) {
                    const int T = gs + t, s = T % kStages;
                    const uint32_t b0_s = b_s + s * 2 * L::kTileB, b1_s = b0_s + L::kTileB;
                    // the tiles arrived long ago; the buffer is what the issue waits for
                    if (!mbar_wait(smem_u32(&bar_full[s]), (T / kStages) & 1, ctl, kBwdBarFull)) { ok = false; break; }
                    if (T >= 2) {
                        // products of step T reuse the TMEM buffer of step T-2
                        if (INPLACE) ok = mbar_wait(smem_u32(&bar_acc[(T - 2) % kStages]), ((T - 2) / kStages) & 1, ctl, kBwdBarAcc);
                        else         ok = mbar_wait(smem_u32(&bar_tfree[g]), ((T >> 1) - 1) & 1, ctl, kBwdBarFree);
                        if (!ok) break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < D / 16; kk++) {
                        const uint32_t offa = (kk >> 2) * L::kBox + (kk & 3) * 32, offb = (kk >> 2) * L::kBoxB + (kk & 3) * 32;
                        mma_f16_ss(tb, make_sdesc(a0_s + offa, hi_k), make_sdesc(b0_s + offb, hi_k), idesc_t, kk > 0);
                    }
#pragma unroll
                    for (int kk = 0; kk < D / 16; kk++) {
                        const uint32_t offa = (kk >> 2) * L::kBox + (kk & 3) * 32, offb = (kk >> 2) * L::kBoxB + (kk & 3) * 32;
                        mma_f16_ss(tb + kW, make_sdesc(a1_s + offa, hi_k), make_sdesc(b1_s + offb, hi_k), idesc_t, kk > 0);
                    }
                    tc_commit(smem_u32(&bar_t[g]));
                    issued = true;
                }
                if (!ok) break;
                // this parity no longer reads the item's stationary tiles once its products are done
                if (issued) tc_commit(smem_u32(&bar_afree[buf]));
                else        mbar_arrive(smem_u32(&bar_afree[buf]));
                gs += it.n_steps;
            }
        }
        __syncwarp();
    } else if (warp == kAccWarp || (warp == kAccWarp + 1 && MODE == 0)) {
        // ------------------------------------------------------------ accumulating MMAs of one accumulator (one thread)
        if (lane == 0) {
            const int x = warp - kAccWarp;
            constexpr uint32_t idesc_acc = make_idesc(kT, D, FMT, FMT, kMajorK, kMajorMN);
            constexpr uint64_t hi_mn = make_sdesc_hi(L::kBoxB, 1024);
            // MODE 0: warp 18 dV += P^T dO (operand P^T, streamed dO = B1), warp 19 dK += dS^T Q (dS^T, Q = B0)
            // MODE 1: warp 18 dQ += dS K (dS, K = B0)
            const bool use_p = (MODE == 0 && x == 0);
            const uint32_t acc = tmem + (x == 0 ? ACC0_COL : ACC1_COL);
            const uint32_t op0 = tmem + (use_p ? OPP0 : OPD0);
            BwdItem it;
            int gs = 0;
            bool ok = true;
            for (int k = 0; ok && bwd_item<CAUSAL, MODE>(k, n_items, n_bh, n_tiles, seq_len, it); k++) {
                for (int t = 0; t < it.n_steps; t++) {
                    const int T = gs + t, s = T % kStages, g = T & 1;
                    const uint32_t bt_s = b_s + s * 2 * L::kTileB + (use_p ? L::kTileB : 0);
                    if (!mbar_wait(smem_u32(&bar_p[g]), (T >> 1) & 1, ctl, kBwdBarP)) { ok = false; break; }
                    // the accumulators of the item before must have been read out
                    if (t == 0 && k >= 1 && !mbar_wait(smem_u32(&bar_accfree), (k - 1) & 1, ctl, kBwdBarFree)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < kW / 16; kk++)
                        mma_f16_ts(acc, op0 + g * OP_STRIDE + op16_col(kk, INPLACE), make_sdesc(bt_s + kk * 2048, hi_mn), idesc_acc,
                                   (t > 0 || kk > 0) ? 1u : 0u);
                    tc_commit(smem_u32(&bar_acc[s]));
                    if (t == it.n_steps - 1) tc_commit(smem_u32(&bar_done));
                }
                gs += it.n_steps;
            }
        }
        __syncwarp();
    } else if (warp == kTmemWarp && STAGED) {
        // ------------------------------------------------------------ TMA stores of the staged output tiles
        BwdItem it;
        for (int k = 0; bwd_item<CAUSAL, MODE>(k, n_items, n_bh, n_tiles, seq_len, it); k++) {
            const int buf = k % NA;
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_ostaged), k & 1, ctl, kBwdBarDone))) break;
            if (lane == 0) {
                const uint32_t o_s = base + buf * 2 * L::kTile;
                for (int b = 0; b < NBOX; b++) {
                    tma_store_3d(&to0, o_s + b * L::kBox, b * 64, it.tile * kT, it.bh);
                    if (MODE == 0) tma_store_3d(&to1, o_s + L::kTile + b * L::kBox, b * 64, it.tile * kT, it.bh);
                }
                tma_store_commit();
                tma_store_wait_read();                      // the buffer may take the stationary tiles of item k + 2
                mbar_arrive(smem_u32(&bar_ofree[buf]));
            }
            __syncwarp();
        }
    } else if (warp < kComputeWarps) {
        // ------------------------------------------------------------ two threads per stationary row and parity
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kBwdRegsCompute));
        const int g = warp >> 3;                            // parity of the steps this warp works on
        const int half = (warp >> 2) & 1;                   // which 32 streamed columns of a step
        const int gt = tid & 255;                           // thread within the parity's warps
        // MODE 0: the streamed column of a step whose statistics this thread stages, and where
        const int st_col = WARP_STATS ? half * 32 + lane : gt;
        const bool st_mine = WARP_STATS || gt < kW;
        const int st_set = (MODE != 0) ? 0 : (WARP_STATS ? warp : g);
        const int st_pair = WARP_STATS ? (lane >> 1) : (gt >> 1) & 31, st_pair0 = WARP_STATS ? 0 : half * 16;
        const int r = tid & (kT - 1);                       // == TMEM lane
        const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const float scale_log2 = scale * kLog2e;
        const uint64_t scale_log2_2 = pack2(scale_log2, scale_log2), scale2 = pack2(scale, scale);
        // The first statistics an item needs are fetched while the item before drains: MODE 1 the
        // LSE and delta of this thread's query row (+inf as LSE makes p = 0), MODE 0 those of the
        // column this thread stages for the parity's first step.
        // `ahead` = 0: MODE 1 this thread's query row, MODE 0 the parity's first step of item x;
        // `ahead` = 1 (MODE 0 only): the parity's second step.
        auto prefetch = [&](const BwdItem& x, int gs_x, int ahead, float& l2, float& dl) {
            const int t = ((g ^ gs_x) & 1) + 2 * ahead;
            const int row = (MODE == 1) ? x.tile * kT + r : x.row0 + t * kW + st_col;
            const bool mine = (MODE == 1) ? (ahead == 0) : (st_mine && t < x.n_steps);
            l2 = INFINITY;
            dl = 0.0f;
            if (mine && row < seq_len) {
                l2 = lse[static_cast<size_t>(x.bh) * seq_len + row] * kLog2e;
                dl = delta[static_cast<size_t>(x.bh) * seq_len + row];
            }
        };
        BwdItem it;
        int gs = 0;
        bool ok = true;
        bool have = bwd_item<CAUSAL, MODE>(0, n_items, n_bh, n_tiles, seq_len, it);
        float pf_l2 = INFINITY, pf_dl = 0.0f, pf2_l2 = INFINITY, pf2_dl = 0.0f;
        if (have) {
            prefetch(it, 0, 0, pf_l2, pf_dl);
            if (MODE == 0) prefetch(it, 0, 1, pf2_l2, pf2_dl);
        }
        for (int k = 0; have; k++) {
            const int tile = it.tile, row0 = it.row0, n_steps = it.n_steps;
            const int r_glob = tile * kT + r;
            const float* lse_h = lse + static_cast<size_t>(it.bh) * seq_len;
            const float* delta_h = delta + static_cast<size_t>(it.bh) * seq_len;
            const float row_lse2 = pf_l2, row_delta = pf_dl;    // MODE 1
            // MODE 0: statistics of the streamed queries, one per column: threads 0..kW-1 of the parity
            // fetch those of its step after next from global memory and stage those of its next step in
            // shared memory while the current ones are in use; rows past the end get LSE = +inf
            auto fetch_stats = [&](int t, float& l2, float& dl) {
                const int qi = row0 + t * kW + st_col;
                l2 = INFINITY;
                dl = 0.0f;
                if (MODE == 0 && st_mine && t < n_steps && qi < seq_len) { l2 = lse_h[qi] * kLog2e; dl = delta_h[qi]; }
            };
            auto stage_stats = [&](int slot, float l2, float dl) {
                if (st_mine) {
                    st_neg[st_set][slot][st_pair][st_col & 1] = -l2;
                    st_neg[st_set][slot][st_pair][2 + (st_col & 1)] = -dl * scale;
                }
            };
            const int t_first = (g ^ gs) & 1;               // this parity's first step of the item
            float nx_l2, nx_dl;
            if (MODE == 0) {
                // the slot of the first step was last read two of this parity's steps ago
                stage_stats(((gs + t_first) >> 1) & 1, pf_l2, pf_dl);
                nx_l2 = pf2_l2;
                nx_dl = pf2_dl;
            }
            const uint64_t row_neg_l2 = pack2(-row_lse2, -row_lse2), row_neg_dl = pack2(-row_delta * scale, -row_delta * scale);
            for (int t = t_first; t < n_steps; t += 2) {
                const int T = gs + t, i = T >> 1;
                const int c0 = row0 + t * kW;               // first streamed row (= column of T0/T1) of the step
                const uint32_t tb = tmem + lane_off + g * 128 + half * 32;
                ok = ok && __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_t[g]), i & 1, ctl, kBwdBarT));
                if (MODE == 0 && !WARP_STATS) {
                    // the parity's warps are past their reads of the other slot; this step's values
                    // (written a step ago) become visible; all eight warps leave together on an abort
                    if (group_sync_or(1 + g, 256, !ok)) { ok = false; break; }
                } else if (!ok) {
                    break;
                }
                if (MODE == 0) {
                    stage_stats((i + 1) & 1, nx_l2, nx_dl);
                    // own staging: every lane is past its reads of that slot (the warp has synchronised
                    // since), and this step's values, written a step ago, are visible from here
                    if (WARP_STATS) __syncwarp();
                    fetch_stats(t + 4, nx_l2, nx_dl);
                }
                tc_fence_after();
                // masking only where the step touches the causal diagonal or the ragged end: masked
                // scores become -inf, so p = 0 and dS = 0
                const bool need_mask = (MODE == 0) ? (CAUSAL && c0 < (tile + 1) * kT)
                                                   : ((CAUSAL && c0 + kW > tile * kT) || c0 + kW > seq_len);
                uint32_t pk[16], dk[16];
#pragma unroll
                for (int c = 0; c < 2; c++) {               // 16 columns of each product at a time
                    uint32_t sv[16], dv[16];
                    tmem_ld16x2_wait(tb + c * 16, sv, tb + kW + c * 16, dv);
                    if (c == 1 && !INPLACE) {
                        // the product buffer is free for this parity's next step
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&bar_tfree[g]));
                    }
                    if (need_mask) {
#pragma unroll
                        for (int e = 0; e < 16; e++) {
                            const int cg = c0 + half * 32 + c * 16 + e;     // global index of the streamed row
                            const bool valid = (MODE == 0) ? (r_glob <= cg) : (cg < seq_len && (!CAUSAL || cg <= r_glob));
                            sv[e] = valid ? sv[e] : 0xff800000u;    // -inf
                        }
                    }
#pragma unroll
                    for (int e = 0; e < 16; e += 2) {
                        uint64_t neg_l2 = row_neg_l2, neg_dl = row_neg_dl;
                        if (MODE == 0) {                    // per column: one 16-byte shared load per pair
                            const float4 st = *reinterpret_cast<const float4*>(st_neg[st_set][i & 1][st_pair0 + c * 8 + (e >> 1)]);
                            neg_l2 = pack2(st.x, st.y);
                            neg_dl = pack2(st.z, st.w);
                        }
                        // p = 2^(s * scale * log2e - lse * log2e);  dS = p * (dP * scale - delta * scale)
                        const uint64_t x = fma2(pack2(__uint_as_float(sv[e]), __uint_as_float(sv[e + 1])), scale_log2_2, neg_l2);
                        float x0, x1;
                        unpack2(x, x0, x1);
                        const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
                        const uint64_t gg = fma2(pack2(__uint_as_float(dv[e]), __uint_as_float(dv[e + 1])), scale2, neg_dl);
                        float e0, e1;
                        unpack2(mul2(pack2(p0, p1), gg), e0, e1);
                        pk[c * 8 + (e >> 1)] = pack_16<BF16>(p0, p1);
                        dk[c * 8 + (e >> 1)] = pack_16<BF16>(e0, e1);
                    }
                }
                if (!INPLACE && T >= 2) {
                    // the operand columns of this parity were read by the accumulations of step T-2
                    if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_acc[(T - 2) % kStages]), ((T - 2) / kStages) & 1, ctl, kBwdBarAcc))) {
                        ok = false;
                        if (MODE == 0 && !WARP_STATS) continue;   // leave with the others at the next rendezvous
                        break;
                    }
                }
                // each half writes its 16 columns of pairs; in place they land on the first half of the
                // 32 columns this thread has read itself
                const uint32_t op_off = INPLACE ? half * 32u : half * 16u;
                if (MODE == 0) tmem_st_x16(tmem + lane_off + OPP0 + g * OP_STRIDE + op_off, pk);
                tmem_st_x16(tmem + lane_off + OPD0 + g * OP_STRIDE + op_off, dk);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar_p[g]));
            }
            if (!ok && (MODE == 1 || WARP_STATS)) break;
            BwdItem nx;
            const bool have_nx = bwd_item<CAUSAL, MODE>(k + 1, n_items, n_bh, n_tiles, seq_len, nx);
            if (have_nx) {
                prefetch(nx, gs + n_steps, 0, pf_l2, pf_dl);
                if (MODE == 0) prefetch(nx, gs + n_steps, 1, pf2_l2, pf2_dl);
            }
            // ---- accumulators -> 16-bit -> global, 32 columns per group of four warps at a time
            ok = ok && __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_done), k & 1, ctl, kBwdBarDone));
            if (ok) {
                tc_fence_after();
#pragma unroll 1
                for (int u = (warp >> 2); u < NACC * (D / 32); u += kComputeWarps / 4) {
                    const int which = u / (D / 32), c = u - which * (D / 32);
                    uint16_t* dst = (which == 0 ? out0 : out1) + (static_cast<size_t>(it.bh) * seq_len + r_glob) * D;
                    uint32_t a[32];
                    tmem_ld32_wait(tmem + lane_off + (which == 0 ? ACC0_COL : ACC1_COL) + c * 32, a);
                    if (STAGED) {
                        // 128-byte rows, 16-byte chunks XORed with the row (the layout the tensor map expects)
                        const uint32_t tile_s = base + (k % NA) * 2 * L::kTile + which * L::kTile;
#pragma unroll
                        for (int g8 = 0; g8 < 4; g8++) {
                            uint32_t w[4];
#pragma unroll
                            for (int j = 0; j < 4; j++)
                                w[j] = pack_16<BF16>(__uint_as_float(a[g8 * 8 + 2 * j]), __uint_as_float(a[g8 * 8 + 2 * j + 1]));
                            const int c16 = c * 4 + g8;   // 16-byte group index in the row
                            const uint32_t addr = tile_s + (c16 >> 3) * L::kBox + r * 128 + (((c16 & 7) ^ (r & 7)) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]),
                                         "r"(w[2]), "r"(w[3]) : "memory");
                        }
                    } else if (r_glob < seq_len) {
                        // 32 bytes per store: a full sector per row, half the write transactions of 16-byte stores
#pragma unroll
                        for (int h8 = 0; h8 < 2; h8++) {
                            uint32_t w[8];
#pragma unroll
                            for (int j = 0; j < 8; j++)
                                w[j] = pack_16<BF16>(__uint_as_float(a[h8 * 16 + 2 * j]), __uint_as_float(a[h8 * 16 + 2 * j + 1]));
                            st_global_v8(dst + c * 32 + h8 * 16, w);
                        }
                    }
                }
                // the next item's accumulations may overwrite the accumulators
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar_accfree));
                if (STAGED) {
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bar_ostaged));
                }
            }
            gs += n_steps;
            it = nx;
            have = have_nx;
        }
    }

    tc_fence_before();
    // The dQ kernel runs as a programmatic dependent of the dK/dV kernel and reads none of its
    // outputs, so it never had to wait for it.  But whatever follows on the stream is ordered after
    // THIS kernel only: every thread waits here, after its own work, until the dK/dV grid has
    // completed and flushed, so that the end of this kernel implies the end of both.
    if (MODE == 1) asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();
    if (warp == kTmemWarp) tmem_dealloc(tmem, 512);
}

template <int D, bool CAUSAL, bool BF16, int MODE>
int launch_bwd(const fa_backward_args& a, DeviceState* st, const CUtensorMap& tq, const CUtensorMap& tk,
               const CUtensorMap& tv, const CUtensorMap& tdo, const CUtensorMap& to0, const CUtensorMap& to1,
               const float* delta, void* out0, void* out1) {
    using L = BwdSmem<D>;
    auto kernel = bwd_kernel<D, CAUSAL, BF16, MODE>;
    static bool configured[64] = {};
    if (!configured[st->device]) {
        FA_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
        configured[st->device] = true;
    }
    const int n_tiles = (a.seq_len + kT - 1) / kT;
    const long long n_bh = (long long)a.batch_size * a.num_heads;
    const long long n_items = n_bh * n_tiles;
    if (n_items > 0x7FFFFFFFll) return FA_ERR_INVALID_ARGUMENT;
    const long long grid = n_items < st->sm_count ? n_items : st->sm_count;   // persistent: one CTA per SM
    // The dQ kernel (MODE 1) reads nothing the dK/dV kernel (MODE 0) writes, so it is launched as a
    // programmatic dependent: its CTAs may start on SMs the first kernel no longer needs (that kernel
    // signals at its start), instead of waiting for its last CTA.  delta comes from a kernel that
    // completed before MODE 0 started.  Before it ends, every thread of the dQ kernel executes
    // griddepcontrol.wait, so later work on the stream (or the next node of a captured graph) sees
    // dK and dV complete as well.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kBwdThreads);
    cfg.dynamicSmemBytes = L::kTotal;
    cfg.stream = static_cast<cudaStream_t>(a.stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (MODE == 1) ? 1 : 0;
    FA_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, tq, tk, tv, tdo, to0, to1, a.lse, delta, static_cast<uint16_t*>(out0),
                                   static_cast<uint16_t*>(out1), a.seq_len, n_tiles, (int)n_bh, (int)n_items, a.scale,
                                   st->status));
    return FA_OK;
}

// maps[0..3]: q, k, v, dO with boxes of 128 rows; maps[4..7]: the same with boxes of kW rows;
// maps[8..10]: dq, dk, dv with boxes of 128 rows
template <int D, bool CAUSAL, bool BF16>
int launch_both(const fa_backward_args& a, DeviceState* st, const CUtensorMap* m, const float* delta) {
    // dK, dV: K and V stay (128-row boxes), Q and dO stream (kW-row boxes)
    int rc = launch_bwd<D, CAUSAL, BF16, 0>(a, st, m[1], m[2], m[4], m[7], m[10], m[9], delta, a.dv, a.dk);
    if (rc != FA_OK) return rc;
    // dQ: Q and dO stay, K and V stream
    return launch_bwd<D, CAUSAL, BF16, 1>(a, st, m[0], m[3], m[5], m[6], m[8], m[8], delta, a.dq, nullptr);
}

}  // namespace
}  // namespace fa

using namespace fa;

FA_EXPORT size_t fa_backward_workspace_bytes(int batch_size, int num_heads, int seq_len) {
    if (batch_size <= 0 || num_heads <= 0 || seq_len <= 0) return 0;
    return (size_t)batch_size * num_heads * seq_len * sizeof(float);
}

FA_EXPORT int fa_backward(const fa_backward_args* a) {
    if (!a || !a->q || !a->k || !a->v || !a->o || !a->d_o || !a->lse || !a->dq || !a->dk || !a->dv)
        return FA_ERR_INVALID_ARGUMENT;
    if (a->batch_size <= 0 || a->num_heads <= 0 || a->seq_len <= 0) return FA_ERR_INVALID_ARGUMENT;
    if (!(a->scale > 0.0f) || !std::isfinite(a->scale)) return FA_ERR_INVALID_ARGUMENT;
    if (a->dtype != FA_DTYPE_F16 && a->dtype != FA_DTYPE_BF16) return FA_ERR_UNSUPPORTED;
    if (a->d_head != 64 && a->d_head != 128) return FA_ERR_UNSUPPORTED;
    const void* ptrs[] = {a->q, a->k, a->v, a->o, a->d_o, a->dq, a->dk, a->dv, a->workspace};
    for (const void* p : ptrs)
        if (!aligned16(p)) return FA_ERR_MISALIGNED;
    const size_t need = fa_backward_workspace_bytes(a->batch_size, a->num_heads, a->seq_len);
    if (!a->workspace || a->workspace_bytes < need) return FA_ERR_WORKSPACE;
    DeviceState* st = device_state();
    if (!st) return FA_ERR_CUDA;
    if (st->cc_major != 10) return FA_ERR_NOT_SM100;

    const uint64_t n_bh = (uint64_t)a->batch_size * a->num_heads;
    const long long n_rows = (long long)n_bh * a->seq_len;
    float* delta = static_cast<float*>(a->workspace);
    cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
    const bool bf = a->dtype == FA_DTYPE_BF16;
    {
        const long long rows_per_block = 8 * (32 / (a->d_head >> 3));      // 8 warps of 4 or 2 rows
        const unsigned blocks = (unsigned)((n_rows + rows_per_block - 1) / rows_per_block);
        if (bf) delta_kernel<true><<<blocks, 256, 0, stream>>>(static_cast<const uint16_t*>(a->o),
                    static_cast<const uint16_t*>(a->d_o), delta, n_rows, a->d_head);
        else    delta_kernel<false><<<blocks, 256, 0, stream>>>(static_cast<const uint16_t*>(a->o),
                    static_cast<const uint16_t*>(a->d_o), delta, n_rows, a->d_head);
        FA_CUDA_TRY(cudaGetLastError());
    }
    CUtensorMap maps[11];
    const void* tensors[4] = {a->q, a->k, a->v, a->d_o};
    int rc;
    for (int i = 0; i < 4; i++) {
        if ((rc = make_tensor_map_3d(&maps[i], tensors[i], a->dtype, a->d_head, a->seq_len, n_bh, 64, kT)) != FA_OK) return rc;
        if ((rc = make_tensor_map_3d(&maps[4 + i], tensors[i], a->dtype, a->d_head, a->seq_len, n_bh, 64, kW)) != FA_OK) return rc;
    }
    void* outs[3] = {a->dq, a->dk, a->dv};
    for (int i = 0; i < 3; i++)
        if ((rc = make_tensor_map_3d(&maps[8 + i], outs[i], a->dtype, a->d_head, a->seq_len, n_bh, 64, kT)) != FA_OK) return rc;
    const bool causal = a->causal != 0;
#define FA_BWD(DH)                                                                              \
    (causal ? (bf ? launch_both<DH, true, true>(*a, st, maps, delta)                             \
                  : launch_both<DH, true, false>(*a, st, maps, delta))                           \
            : (bf ? launch_both<DH, false, true>(*a, st, maps, delta)                            \
                  : launch_both<DH, false, false>(*a, st, maps, delta)))
    if (a->d_head == 64) return FA_BWD(64);
    return FA_BWD(128);
#undef FA_BWD
}
