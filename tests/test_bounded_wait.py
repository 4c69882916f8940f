"""CPU unit test of the give-up rule every spin-wait of the kernels follows.

``tensorax_b200/csrc/bounded_wait.h`` holds the rule as a template over its probes; the kernels instantiate it
with PTX (mbarrier.test_wait / try_wait, %globaltimer), this test compiles it as plain C++ with scripted probes
and a fake clock.  (What it replaces in the reference: CUDA_CHECK's print-and-exit, csrc/cuda/cuda_utils.cuh:6-14;
the reference's kernels themselves have no failure path.)"""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROGRAM = r'''
#include <cstdio>
#include "bounded_wait.h"
using namespace txb;
struct Script {
    long polls = 0, ready_after = -1;      // the phase completes at this poll (-1: never)
    uint64_t clock = 1000, tick = 50;      // fake nanosecond clock, advanced per reading
    long clock_reads = 0;
};
static bool run(Script &s, volatile int *abort_flag, uint64_t limit, bool quick_hit = false)
{
    return bounded_wait([&] { return quick_hit; },
                        [&] { ++s.polls; return s.ready_after >= 0 && s.polls >= s.ready_after; },
                        [&] { ++s.clock_reads; s.clock += s.tick; return s.clock; }, abort_flag, limit);
}
int main()
{
    int fails = 0;
    volatile int flag = 0;
    { Script s; bool r = run(s, &flag, 1000, true);                       // already complete: no poll, no clock
      if (!(r && s.polls == 0 && s.clock_reads == 0)) { printf("case quick failed\n"); ++fails; } }
    { Script s; s.ready_after = 5; bool r = run(s, &flag, 1000);          // completes before the first check
      if (!(r && s.polls == 5 && s.clock_reads == 0)) { printf("case early failed\n"); ++fails; } }
    { Script s; s.ready_after = 1000; bool r = run(s, &flag, 1000000);    // completes after several checks, inside the limit
      if (!(r && s.polls == 1000 && s.clock_reads == 1000 / (long)kWaitCheckEvery)) { printf("case late failed %ld %ld\n", s.polls, s.clock_reads); ++fails; } }
    { Script s; s.tick = 400; bool r = run(s, &flag, 1000);               // never completes: gives up once the clock has moved past the limit
      // first check only starts the clock; checks 2..4 see 400, 800, 1200 ns elapsed -> false at the 4th check
      if (!(!r && s.clock_reads == 4 && s.polls == 4 * (long)kWaitCheckEvery)) { printf("case timeout failed %ld %ld\n", s.polls, s.clock_reads); ++fails; } }
    { Script s; flag = 1; bool r = run(s, &flag, ~0ull);                  // somebody else gave up: stop at the next check, whatever the clock says
      if (!(!r && s.polls == (long)kWaitCheckEvery && s.clock_reads == 0)) { printf("case abort failed %ld %ld\n", s.polls, s.clock_reads); ++fails; } flag = 0; }
    { Script s; s.ready_after = (long)kWaitCheckEvery; flag = 1; bool r = run(s, &flag, 10);   // completion wins over a raised flag seen in the same round
      if (!r) { printf("case completion-first failed\n"); ++fails; } flag = 0; }
    printf(fails ? "FAILED\n" : "all cases ok\n");
    return fails;
}
'''


def test_bounded_wait_rule_on_cpu(tmp_path):
    src = tmp_path / "bounded_wait_test.cpp"
    exe = tmp_path / "bounded_wait_test"
    src.write_text(PROGRAM)
    inc = os.path.join(ROOT, "tensorax_b200", "csrc")
    cc = subprocess.run(["g++", "-std=c++17", "-O1", "-I", inc, str(src), "-o", str(exe)], capture_output=True, text=True)
    assert cc.returncode == 0, cc.stderr[-3000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert run.returncode == 0 and "all cases ok" in run.stdout, run.stdout + run.stderr


def test_the_kernels_use_that_rule():
    """Every mbarrier wait goes through ptx::mbar_wait, which is bounded_wait with the PTX probes."""
    ptx = open(os.path.join(ROOT, "tensorax_b200", "csrc", "ptx.cuh")).read()
    assert '#include "bounded_wait.h"' in ptx and "return bounded_wait(" in ptx
    for name in ("sdpa_tc.cuh", "sdpa_tc_pair.cuh", "sdpa_bwd.cuh", "linear_tc.cuh"):
        text = open(os.path.join(ROOT, "tensorax_b200", "csrc", name)).read()
        assert "mbar_wait(" in text
        assert "__trap" not in text and "assert(" not in text.replace("static_assert(", "")
