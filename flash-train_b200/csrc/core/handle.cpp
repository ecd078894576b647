#include "core/handle.hpp"

#include <mutex>
#include <utility>

namespace ftrain {

void Handle::registerOpsEngine(std::shared_ptr<OpsEngineBase> engine) {
    if (engine == nullptr) { throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "OpsEngine must not be null"); }
    const std::unique_lock<std::shared_mutex> lock(mutex_);
    PatternKey key = engine->getPattern().getKey();
    if (!engines_.emplace(std::move(key), std::move(engine)).second) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "An OpsEngine is already registered for this PatternKey");
    }
}

std::shared_ptr<const OpsEngineBase> Handle::findOpsEngine(const PatternKey& key) const {
    const std::shared_lock<std::shared_mutex> lock(mutex_);
    const auto found = engines_.find(key);
    return found == engines_.end() ? nullptr : found->second;
}

std::size_t Handle::getNumOpsEngines() const {
    const std::shared_lock<std::shared_mutex> lock(mutex_);
    return engines_.size();
}

Handle& getGlobalHandle() {
    // Built-ins are in place before any caller can observe the registry.
    static Handle* const handle = [] {
        auto* created = new Handle();
        for (auto& engine : makeBuiltinOpsEngines()) { created->registerOpsEngine(std::move(engine)); }
        return created;
    }();
    return *handle;
}

}  // namespace ftrain
