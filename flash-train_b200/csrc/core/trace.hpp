// Trace ranges for profilers: NVTX on this platform (the reference uses ROCTX,
// src/trace.cpp:14-36). Neither call throws; with no profiler attached a range
// costs one indirect call that returns immediately.
#ifndef FTRAIN_CORE_TRACE_HPP_
#define FTRAIN_CORE_TRACE_HPP_

namespace ftrain {

class ScopedTraceRange final {
  public:
    explicit ScopedTraceRange(const char* name) noexcept;
    ~ScopedTraceRange() noexcept;
    ScopedTraceRange(const ScopedTraceRange&)            = delete;
    ScopedTraceRange& operator=(const ScopedTraceRange&) = delete;

  private:
    bool active_{false};
};

void markTraceEvent(const char* name) noexcept;

}  // namespace ftrain

#endif
