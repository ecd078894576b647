#include "core/trace.hpp"

#include "ftcuda/ftcuda.h"

namespace ftrain {

ScopedTraceRange::ScopedTraceRange(const char* name) noexcept : active_(ftcuda_trace_push(name) != 0) {}

ScopedTraceRange::~ScopedTraceRange() noexcept {
    if (active_) { ftcuda_trace_pop(); }
}

void markTraceEvent(const char* name) noexcept { ftcuda_trace_mark(name); }

}  // namespace ftrain
