// The give-up rule every spin-wait of the kernels follows, written so that it also compiles as
// plain C++ for the CPU unit test (tests/test_bounded_wait.py): the kernels pass PTX probes
// (mbarrier.test_wait / try_wait, %globaltimer), the test passes scripted ones.
//
// This replaces the reference's error handling on the device path -- its launchers print and
// exit() on a CUDA error (tensorax csrc/cuda/cuda_utils.cuh:6-14) and its kernels cannot fail
// softly at all -- with: a wait ends when the awaited phase completes (true), when another
// thread of the CTA has already given up (false), or when `limit_ns` of wall-clock time have
// passed since the first slow-path check (false).  The bound is wall-clock because one
// try_wait may itself suspend the thread for a hardware-chosen time.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define TX_HD __host__ __device__ __forceinline__
#else
#define TX_HD inline
#endif

namespace txb {

constexpr uint64_t kWaitLimitNs = 2000000000ull;   // 2 s: far beyond any legitimate wait of these kernels
constexpr uint32_t kWaitCheckEvery = 128;          // polls between two looks at the abort flag and the clock

// quick():   non-blocking probe, true = the phase is over        (the common case, tried once first)
// blocking(): probe that may park the thread for a while, true = the phase is over
// now():     nanosecond clock
template <class Quick, class Blocking, class Clock>
TX_HD bool bounded_wait(Quick quick, Blocking blocking, Clock now, volatile int *abort_flag, uint64_t limit_ns)
{
    if (quick()) return true;
    uint64_t t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (blocking()) return true;
        if ((i % kWaitCheckEvery) == kWaitCheckEvery - 1) {
            if (*abort_flag) return false;
            const uint64_t t = now();
            if (t0 == 0) t0 = t;
            else if (t - t0 > limit_ns) return false;
        }
    }
}

}  // namespace txb
