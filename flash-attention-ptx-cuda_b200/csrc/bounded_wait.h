// The decision core of every device-side wait, kept free of device-only
// instructions so that the same code runs on the host: a unit test drives it
// with a poll that never succeeds and a fake clock, which is the only way the
// give-up branch is ever exercised (no test makes a GPU wait run out).
//
// The reference has no counterpart: its kernel synchronises with block-wide
// barriers only (kernels/flash_attention.cu:349,396,470) and its launcher
// reports errors by printing and exiting (include/flash_attention.h:35-43).
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define FA_HOST_DEVICE __host__ __device__ __forceinline__
#else
#define FA_HOST_DEVICE inline
#endif

namespace fa {

// Error words written to the device status buffer: (code << 16) | detail.
enum : int {
    kErrNone        = 0,
    kErrWaitTimeout = 1,   // a bounded wait ran out of time; detail = barrier id
};

enum : int { kWaitDone = 0, kWaitAborted = 1, kWaitTimedOut = 2 };

// Polls until `poll()` returns true.  Every `check_every` polls (a power of two) it looks at
// `aborted()` - somebody else in the CTA already gave up - and at the clock `now_ns()`; the
// wait gives up once more than `limit_ns` have passed since its first look at the clock.
template <class Poll, class Aborted, class Clock>
FA_HOST_DEVICE int bounded_wait(Poll poll, Aborted aborted, Clock now_ns, unsigned long long limit_ns,
                                uint32_t check_every) {
    unsigned long long t0 = 0;
    bool have_t0 = false;
    uint32_t polls = 0;
    while (!poll()) {
        if ((++polls & (check_every - 1u)) == 0u) {
            if (aborted()) return kWaitAborted;
            const unsigned long long now = now_ns();
            if (!have_t0) {
                t0 = now;
                have_t0 = true;
            } else if (now - t0 > limit_ns) {
                return kWaitTimedOut;
            }
        }
    }
    return kWaitDone;
}

// The status word a waiter records when it gives up on barrier `barrier_id`.
FA_HOST_DEVICE int wait_timeout_word(int barrier_id) { return (kErrWaitTimeout << 16) | (barrier_id & 0xFFFF); }

// Host side: what a status word read back from the device means for the caller.
// 0 -> 0 (FA_OK); a recorded wait timeout -> -6 (FA_ERR_DEVICE_TIMEOUT); any other
// non-zero word is reported the same way (a kernel recorded an error and stopped early).
FA_HOST_DEVICE int status_word_to_error(int word) { return word == 0 ? 0 : -6; }
FA_HOST_DEVICE int status_word_code(int word) { return (word >> 16) & 0xFFFF; }
FA_HOST_DEVICE int status_word_detail(int word) { return word & 0xFFFF; }

}  // namespace fa
