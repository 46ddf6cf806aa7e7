// Host-side driver of fa::bounded_wait (csrc/bounded_wait.h): the give-up branch of the device-side
// waits, exercised with polls that never succeed and a fake clock.  Prints "ok" and exits 0, or
// prints what failed and exits 1.  Built and run by tests/test_bounded_wait_cpu.py.
#include <cstdio>
#include <cstdlib>

#include "bounded_wait.h"

#define CHECK(cond)                                                        \
    do {                                                                   \
        if (!(cond)) { std::printf("FAILED line %d: %s\n", __LINE__, #cond); return 1; } \
    } while (0)

int main() {
    using namespace fa;
    const unsigned long long limit = 2000000000ull;        // 2 s, the device-side limit

    // 1. a poll that never succeeds: the wait must give up once the fake clock has moved past the limit
    {
        unsigned long long clock = 5, polls = 0, looks = 0;
        const int r = bounded_wait([&] { polls++; return false; }, [] { return false; },
                                   [&] { looks++; clock += 300000000ull; return clock; }, limit, 16u);
        CHECK(r == kWaitTimedOut);
        // first look starts the stopwatch; it then takes 7 more looks of 0.3 s to exceed 2 s
        CHECK(looks == 8);
        CHECK(polls == 8 * 16);                             // the clock is read every 16th poll only
    }
    // 2. a clock that starts at 0 must still start the stopwatch at its first look
    {
        unsigned long long clock = 0, looks = 0;
        const int r = bounded_wait([] { return false; }, [] { return false; },
                                   [&] { const unsigned long long now = clock; clock += limit + 1; looks++; return now; },
                                   limit, 4u);
        CHECK(r == kWaitTimedOut && looks == 2);
    }
    // 3. somebody else in the CTA gave up: leave at the next look, without reading the clock again
    {
        int polls = 0, looks = 0;
        bool abort_flag = false;
        const int r = bounded_wait([&] { if (++polls == 40) abort_flag = true; return false; },
                                   [&] { return abort_flag; }, [&] { looks++; return 1ull; }, limit, 16u);
        CHECK(r == kWaitAborted);
        CHECK(polls == 48 && looks == 2);                   // looks at polls 16 and 32; abort seen at poll 48
    }
    // 4. the awaited thing happens: no time-out however long it took in polls, as long as the clock is within the limit
    {
        int polls = 0;
        unsigned long long clock = 0;
        const int r = bounded_wait([&] { return ++polls == 1000; }, [] { return false; },
                                   [&] { clock += 1000; return clock; }, limit, 16u);
        CHECK(r == kWaitDone && polls == 1000);
    }
    // 5. success on the first poll never touches the clock or the abort flag
    {
        int looks = 0;
        const int r = bounded_wait([] { return true; }, [&] { looks++; return true; }, [&] { looks++; return 0ull; },
                                   limit, 16u);
        CHECK(r == kWaitDone && looks == 0);
    }
    // 6. the words a waiter records and what the host makes of them
    CHECK(wait_timeout_word(0x41) == ((1 << 16) | 0x41));
    CHECK(status_word_code(wait_timeout_word(7)) == kErrWaitTimeout && status_word_detail(wait_timeout_word(7)) == 7);
    CHECK(status_word_to_error(0) == 0);
    CHECK(status_word_to_error(wait_timeout_word(3)) == -6);
    std::printf("ok\n");
    return 0;
}
