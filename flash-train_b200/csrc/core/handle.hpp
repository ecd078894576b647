// Process-wide registry: PatternKey -> engine. Entries are never replaced or
// removed. Reference: src/include/flash_train/handle.hpp:19-38, src/handle.cpp:36-61.
#ifndef FTRAIN_CORE_HANDLE_HPP_
#define FTRAIN_CORE_HANDLE_HPP_

#include <cstddef>
#include <memory>
#include <shared_mutex>
#include <unordered_map>

#include "core/engine.hpp"

namespace ftrain {

class Handle final {
  public:
    // A null engine or an already-registered key throws
    // Exception(FTRAIN_STATUS_INVALID_ARGUMENT).
    void registerOpsEngine(std::shared_ptr<OpsEngineBase> engine);
    // Empty pointer when nothing is registered for the key.
    std::shared_ptr<const OpsEngineBase> findOpsEngine(const PatternKey& key) const;
    std::size_t getNumOpsEngines() const;

  private:
    mutable std::shared_mutex mutex_;
    std::unordered_map<PatternKey, std::shared_ptr<const OpsEngineBase>, PatternKeyHasher> engines_;
};

// The registry with every built-in engine already in it; the first call
// registers them (thread-safe).
Handle& getGlobalHandle();

}  // namespace ftrain

#endif
