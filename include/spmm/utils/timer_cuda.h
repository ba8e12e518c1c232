// Event timer and iteration counts of the reference's harness (include/spmm/utils/timer_cuda.h:3-40),
// over the C ABI's events.  Same names, same 20 warm-up / 200 timed launches.
#pragma once
#include "starml/basic/matrix.h"

#define WARMUP_NUM_CUDA 20
#define EXE_NUM_CUDA 200

struct GpuTimer {
  hpspmm_ctx* ctx;
  hpspmm_event start;
  hpspmm_event stop;
  hpspmm_stream stream;

  explicit GpuTimer(hpspmm_stream s = nullptr, int device = 0) : ctx(hpspmm::context(device)), stream(s) {
    hpspmm::check(hpspmm_event_create(ctx, &start), "event_create");
    hpspmm::check(hpspmm_event_create(ctx, &stop), "event_create");
  }
  ~GpuTimer() {
    hpspmm_event_destroy(ctx, start);
    hpspmm_event_destroy(ctx, stop);
  }
  GpuTimer(const GpuTimer&) = delete;
  GpuTimer& operator=(const GpuTimer&) = delete;

  void Start() { hpspmm::check(hpspmm_event_record(ctx, start, stream), "event_record"); }
  void Stop() { hpspmm::check(hpspmm_event_record(ctx, stop, stream), "event_record"); }
  float Elapsed() {
    float ms = 0.f;
    hpspmm::check(hpspmm_event_elapsed_ms(ctx, start, stop, &ms), "event_elapsed");
    return ms;
  }
};
