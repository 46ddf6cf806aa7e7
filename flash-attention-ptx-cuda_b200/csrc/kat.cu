// Tensor-core known-answer test for the tcgen05 path.
//
// The reference gates its attention tests behind an instruction-level check of
// its mma.sync + ldmatrix addressing (src/bench.cu:51-165, test_ptx_mma: A = I,
// B = a counting pattern, expect C == B).  This file is the same idea for the
// machinery the sm_100a kernels rely on: TMA tensor maps with 128-byte swizzle,
// UMMA shared-memory descriptors (K-major Q and K, MN-major V), the TMEM layout
// of a 16-bit A operand written with tcgen05.st, instruction descriptors, and
// tcgen05.ld of the fp32 accumulators.  One CTA computes
//     S = Q K^T,   P = round16(S * p_scale),   O = P V
// on a single 128 x 128 x d_head tile and returns S and O, which the host test
// compares with a CPU product (exactly, for the identity/counting pattern).
#include "host_common.h"
#include "ptx.cuh"

namespace fa {
namespace {

constexpr int kBoxBytes = 128 * 128;   // one TMA box: 128 rows x 128 bytes

template <int D, bool BF16>
__global__ void __launch_bounds__(128)
kat_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
           const __grid_constant__ CUtensorMap tm_v, float* __restrict__ s_out,
           float* __restrict__ o_out, float p_scale, int* status) {
    constexpr int NBOX  = D / 64;
    constexpr int S_COL = 0;
    constexpr int O_COL = 128;
    constexpr int P_COL = (D == 64) ? 192 : 0;   // D = 128: P overwrites the S columns it replaces
    constexpr uint32_t FMT = BF16 ? kFmtBF16 : kFmtF16;

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[3];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_s = base;
    const uint32_t k_s = q_s + NBOX * kBoxBytes;
    const uint32_t v_s = k_s + NBOX * kBoxBytes;
    const int tid = threadIdx.x, warp = tid >> 5;
    WaitCtl ctl{&abort_flag, status};

    if (tid == 0) {
        for (int i = 0; i < 3; i++) mbar_init(smem_u32(&bars[i]), 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();
    if (warp == 0) tmem_alloc(smem_u32(&tmem_slot), 256);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;

    if (tid == 0) {
        mbar_arrive_expect_tx(smem_u32(&bars[0]), 3 * NBOX * kBoxBytes);
        for (int b = 0; b < NBOX; b++) {
            tma_load_3d(q_s + b * kBoxBytes, &tm_q, smem_u32(&bars[0]), b * 64, 0, 0);
            tma_load_3d(k_s + b * kBoxBytes, &tm_k, smem_u32(&bars[0]), b * 64, 0, 0);
            tma_load_3d(v_s + b * kBoxBytes, &tm_v, smem_u32(&bars[0]), b * 64, 0, 0);
        }
    }
    bool ok = mbar_wait(smem_u32(&bars[0]), 0, ctl, 0);

    if (ok && tid == 0) {
        tc_fence_after();
        constexpr uint32_t idesc = make_idesc(128, 128, FMT, FMT, kMajorK, kMajorK);
        constexpr uint64_t hi = make_sdesc_hi(16, 1024);
        for (int kk = 0; kk < D / 16; kk++) {
            const uint32_t off = (kk >> 2) * kBoxBytes + (kk & 3) * 32;
            mma_f16_ss(tmem + S_COL, make_sdesc(q_s + off, hi), make_sdesc(k_s + off, hi), idesc, kk > 0);
        }
        tc_commit(smem_u32(&bars[1]));
    }
    ok = ok && mbar_wait(smem_u32(&bars[1]), 0, ctl, 1);
    tc_fence_after();

    if (ok) {
#pragma unroll 1
        for (int c = 0; c < 4; c++) {
            uint32_t r[32];
            tmem_ld_x32(tmem + lane_off + S_COL + c * 32, r);
            tmem_wait_ld();
            uint32_t p[16];
#pragma unroll
            for (int i = 0; i < 32; i++) s_out[tid * 128 + c * 32 + i] = __uint_as_float(r[i]);
#pragma unroll
            for (int i = 0; i < 16; i++)
                p[i] = pack_16<BF16>(__uint_as_float(r[2 * i]) * p_scale,
                                     __uint_as_float(r[2 * i + 1]) * p_scale);
            tmem_st_x16(tmem + lane_off + P_COL + c * 16, p);
        }
        tmem_wait_st();
    }
    tc_fence_before();
    __syncthreads();

    if (ok && tid == 0) {
        tc_fence_after();
        constexpr uint32_t idesc = make_idesc(128, D, FMT, FMT, kMajorK, kMajorMN);
        constexpr uint64_t hi = make_sdesc_hi(kBoxBytes, 1024);
        for (int kk = 0; kk < 128 / 16; kk++)
            mma_f16_ts(tmem + O_COL, tmem + P_COL + kk * 8, make_sdesc(v_s + kk * 2048, hi), idesc, kk > 0);
        tc_commit(smem_u32(&bars[2]));
    }
    ok = ok && mbar_wait(smem_u32(&bars[2]), 0, ctl, 2);
    tc_fence_after();

    if (ok) {
#pragma unroll 1
        for (int c = 0; c < D / 32; c++) {
            uint32_t r[32];
            tmem_ld_x32(tmem + lane_off + O_COL + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; i++) o_out[tid * D + c * 32 + i] = __uint_as_float(r[i]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

template <int D, bool BF16>
int run_kat(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, float* s_out,
            float* o_out, float p_scale, int* status) {
    const int smem = 3 * (D / 64) * kBoxBytes + 1024;
    FA_CUDA_TRY(cudaFuncSetAttribute(kat_kernel<D, BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kat_kernel<D, BF16><<<1, 128, smem>>>(tq, tk, tv, s_out, o_out, p_scale, status);
    FA_CUDA_TRY(cudaGetLastError());
    return FA_OK;
}

}  // namespace
}  // namespace fa

using namespace fa;

FA_EXPORT int fa_kat(int dtype, int d_head, const void* q_host, const void* k_host,
                     const void* v_host, float p_scale, float* s_out_host, float* o_out_host) {
    if (!q_host || !k_host || !v_host || !s_out_host || !o_out_host) return FA_ERR_INVALID_ARGUMENT;
    if (dtype != FA_DTYPE_F16 && dtype != FA_DTYPE_BF16) return FA_ERR_UNSUPPORTED;
    if (d_head != 64 && d_head != 128) return FA_ERR_UNSUPPORTED;
    DeviceState* st = device_state();
    if (!st) return FA_ERR_CUDA;
    if (st->cc_major != 10) return FA_ERR_NOT_SM100;
    const size_t in_b = (size_t)128 * d_head * 2;
    uint8_t* dev = nullptr;
    const size_t total = 3 * in_b + (size_t)128 * 128 * 4 + (size_t)128 * d_head * 4;
    FA_CUDA_TRY(cudaMalloc(&dev, total));
    uint8_t* dq = dev;
    uint8_t* dk = dq + in_b;
    uint8_t* dv = dk + in_b;
    float* ds = reinterpret_cast<float*>(dv + in_b);
    float* dout = ds + 128 * 128;
    int rc = FA_OK;
    auto fail = [&](int code) { cudaFree(dev); return code; };
    if (cudaMemcpy(dq, q_host, in_b, cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemcpy(dk, k_host, in_b, cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemcpy(dv, v_host, in_b, cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemset(ds, 0, (size_t)128 * 128 * 4 + (size_t)128 * d_head * 4) != cudaSuccess)
        return fail(note_cuda_error(cudaGetLastError(), "fa_kat upload"));
    CUtensorMap tq, tk, tv;
    if ((rc = make_tensor_map_3d(&tq, dq, dtype, d_head, 128, 1, 64, 128)) != FA_OK) return fail(rc);
    if ((rc = make_tensor_map_3d(&tk, dk, dtype, d_head, 128, 1, 64, 128)) != FA_OK) return fail(rc);
    if ((rc = make_tensor_map_3d(&tv, dv, dtype, d_head, 128, 1, 64, 128)) != FA_OK) return fail(rc);
    const bool bf = dtype == FA_DTYPE_BF16;
    if (d_head == 64)
        rc = bf ? run_kat<64, true>(tq, tk, tv, ds, dout, p_scale, st->status)
                : run_kat<64, false>(tq, tk, tv, ds, dout, p_scale, st->status);
    else
        rc = bf ? run_kat<128, true>(tq, tk, tv, ds, dout, p_scale, st->status)
                : run_kat<128, false>(tq, tk, tv, ds, dout, p_scale, st->status);
    if (rc != FA_OK) return fail(rc);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail(note_cuda_error(e, "fa_kat kernel"));
    if (cudaMemcpy(s_out_host, ds, (size_t)128 * 128 * 4, cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(o_out_host, dout, (size_t)128 * d_head * 4, cudaMemcpyDeviceToHost) != cudaSuccess)
        return fail(note_cuda_error(cudaGetLastError(), "fa_kat download"));
    int word = 0;
    if (cudaMemcpy(&word, st->status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
        return fail(note_cuda_error(cudaGetLastError(), "fa_kat status"));
    cudaFree(dev);
    return word == 0 ? FA_OK : FA_ERR_DEVICE_TIMEOUT;
}
