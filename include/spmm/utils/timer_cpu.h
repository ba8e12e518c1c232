// Wall-clock timer and CPU iteration counts (reference: include/spmm/utils/timer_cpu.h:4-28).
#pragma once
#include <chrono>

#define WARMUP_NUM_CPU 2
#define EXE_NUM_CPU 2

struct CpuTimer {
  std::chrono::steady_clock::time_point t0, t1;
  void Start() { t0 = std::chrono::steady_clock::now(); }
  void Stop() { t1 = std::chrono::steady_clock::now(); }
  // milliseconds, like GpuTimer::Elapsed
  float Elapsed() const { return std::chrono::duration<float, std::milli>(t1 - t0).count(); }
};
