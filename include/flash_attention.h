#pragma once
// C++ launch interface of the B200 flash-attention library.
//
// Source compatible with the reference project's include/flash_attention.h
// (struct transformer::FlashAttentionParams at :51-64, launch_flash_attention
// at :67, CUDA_CHECK at :34-44): programs written against that header, such as
// its src/bench.cu and src/demo.cu, compile unchanged against this one and link
// against libfa_b200.so.
//
//   transformer::FlashAttentionParams p = {};
//   p.Q = dQ; p.K = dK; p.V = dV; p.O = dO; p.L = dL;      // device pointers
//   p.batch_size = B; p.num_heads = H; p.seq_len = S; p.d_head = 64;
//   p.scale = 1.0f / sqrtf(64.0f); p.causal = true; p.stream = 0;
//   transformer::launch_flash_attention(p);
//
// Differences from the reference implementation behind the same interface:
//   * d_head is honoured (64 or 128) instead of being ignored;
//   * any seq_len >= 1 works, the (b,h) count is not limited to 65535;
//   * the members after `stream` are additions; value-initialisation (`= {}`)
//     leaves them zero, which means "fp16, no extras" - the legacy behaviour.
// Errors keep the reference's semantics for this entry point: a message on
// stderr and exit(EXIT_FAILURE).  The C ABI in fa_b200.h returns codes instead.

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#ifndef CUDA_CHECK
#define CUDA_CHECK(call)                                                              \
    do {                                                                              \
        cudaError_t fa_cuda_check_err_ = (call);                                      \
        if (fa_cuda_check_err_ != cudaSuccess) {                                      \
            fprintf(stderr, "CUDA error at %s:%d: %s\n", __FILE__, __LINE__,          \
                    cudaGetErrorString(fa_cuda_check_err_));                          \
            exit(EXIT_FAILURE);                                                       \
        }                                                                             \
    } while (0)
#endif

namespace transformer {

struct FlashAttentionParams {
    // ---- members of the reference struct, same names, types and order ----
    const half*  Q;            // [B*H, S, D]
    const half*  K;            // [B*H, S, D]
    const half*  V;            // [B*H, S, D]
    half*        O;            // [B*H, S, D]
    float*       L;            // [B*H, S] natural-log LSE, optional (nullptr)
    int          batch_size;
    int          num_heads;
    int          seq_len;
    int          d_head;       // 64 or 128
    float        scale;        // > 0, typically 1/sqrt(d_head)
    bool         causal;
    cudaStream_t stream;
    // ---- additions; zero = legacy behaviour ----
    int          dtype;        // 0 fp16 (default), 1 bf16 (Q,K,V,O then point at bf16 data)
};

// Enqueues the forward pass on params.stream and returns without synchronising.
void launch_flash_attention(const FlashAttentionParams& params);

}  // namespace transformer
