// OpsEngine: turns Args into an ordered list of configured Primitives.
//
// The selection algorithm is the reference's (src/include/flash_train/engine.hpp:110-242,
// pinned by tests/engine/engine_test.cpp:276-555):
//   1. Args must carry this engine's PatternKey and be complete.
//   2. The family builds and validates its Problem.
//   3. Cache lookup on (constraints tokens, problem tokens). A hit reproduces
//      the cached record order and skips Finders and applicability checks.
//   4. On a miss the Finders are asked in template order; the first Finder
//      that names at least one applicable record supplies the WHOLE selection
//      (its other applicable names follow in its order). Finder names that
//      match no record are ignored; Finders disabled by FTRAIN_DISABLED_FINDERS
//      are not asked. If no Finder contributes, every applicable record
//      follows in registration order; a record already rejected is not
//      re-checked. Records filtered by FTRAIN_ENABLED/DISABLED_PRIMITIVES drop
//      out silently. Nothing applicable -> FTRAIN_STATUS_UNSUPPORTED listing
//      "<name>: <reason>" for each rejection.
//   5. The selection is published to the cache and each selected prototype is
//      cloned and configured for this problem.
//
// A family plugs in through static functions:
//   Family::Problem                                  (with getProblemKey())
//   static Pattern Family::makePattern()
//   static std::vector<std::shared_ptr<const Primitive<Problem>>> Family::makeRecords()
//   static Problem Family::makeProblem(const Args&)
// and each Finder through
//   static const char* Finder::getName()
//   static std::vector<std::string> Finder::findCandidates(const Problem&, const Constraints&)
#ifndef FTRAIN_CORE_ENGINE_HPP_
#define FTRAIN_CORE_ENGINE_HPP_

#include <cstddef>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "core/cache.hpp"
#include "core/constraints.hpp"
#include "core/ops_args.hpp"
#include "core/plan.hpp"
#include "core/primitive.hpp"

namespace ftrain {

class OpsEngineBase {
  public:
    virtual ~OpsEngineBase();
    OpsEngineBase(const OpsEngineBase&)            = delete;
    OpsEngineBase& operator=(const OpsEngineBase&) = delete;

    const Pattern& getPattern() const noexcept { return pattern_; }

    // Safe for concurrent calls with distinct Args.
    virtual std::vector<std::unique_ptr<PrimitiveBase>> createPrimitives(const Args& args,
                                                                         const Constraints& constraints) const = 0;

    // createPrimitives() on the calling thread's current device, wrapped in a
    // Plan bound to that device.
    Plan createPlan(const Args& args) const;

  protected:
    explicit OpsEngineBase(Pattern pattern);

  private:
    Pattern pattern_;
};

template<typename Family, typename... Finders>
class OpsEngine final : public OpsEngineBase {
  public:
    using Problem = typename Family::Problem;
    using Record  = std::shared_ptr<const Primitive<Problem>>;

    // A null record, a null name or a repeated name throws
    // Exception(FTRAIN_STATUS_INVALID_ARGUMENT).
    OpsEngine() : OpsEngineBase(Family::makePattern()), records_(Family::makeRecords()) {
        for (std::size_t i = 0; i < records_.size(); ++i) {
            if (records_[i] == nullptr) {
                throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "OpsEngine Primitive %zu must not be null", i);
            }
            const char* name = records_[i]->getName();
            if (name == nullptr) {
                throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "OpsEngine Primitive %zu must not return a null name", i);
            }
            if (!position_of_.emplace(name, i).second) {
                throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "OpsEngine Primitive %zu repeats the name %s", i, name);
            }
        }
    }

    std::vector<std::unique_ptr<PrimitiveBase>> createPrimitives(const Args& args,
                                                                 const Constraints& constraints) const override {
        if (args.getPatternKey() != getPattern().getKey()) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Args PatternKey does not match this OpsEngine");
        }
        if (!args.isComplete()) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Args has one or more unset Operand or Op parameters");
        }
        const Problem problem = Family::makeProblem(args);
        const CacheKey key(constraints.getConstraintsKey(), problem.getProblemKey());
        if (!isSelectionCacheDisabled()) {
            if (const auto cached = cache_.find(key)) { return instantiate(*cached, problem); }
        }
        return instantiate(select(problem, constraints, key), problem);
    }

    std::size_t getCacheSize() const { return cache_.getSize(); }

  private:
    // Bookkeeping of one selection walk.
    struct Walk {
        std::vector<std::size_t> chosen;
        std::vector<bool> offered;
        std::string rejections;
    };

    std::vector<std::size_t> select(const Problem& problem, const Constraints& constraints, const CacheKey& key) const {
        Walk walk;
        walk.offered.assign(records_.size(), false);
        const bool by_finder = (askFinder<Finders>(problem, constraints, walk) || ...);
        if (!by_finder) {
            for (std::size_t i = 0; i < records_.size(); ++i) { offer(i, problem, constraints, walk); }
        }
        if (walk.chosen.empty()) {
            throw Exception(FTRAIN_STATUS_UNSUPPORTED,
                            "No Primitive supports the supplied Args and runtime constraints (%s)",
                            walk.rejections.c_str());
        }
        cache_.publish(key, walk.chosen);
        return std::move(walk.chosen);
    }

    template<typename Finder>
    bool askFinder(const Problem& problem, const Constraints& constraints, Walk& walk) const {
        if (isFinderDisabled(Finder::getName())) { return false; }
        bool contributed = false;
        for (const std::string& name : Finder::findCandidates(problem, constraints)) {
            const auto found = position_of_.find(name);
            if (found == position_of_.end()) { continue; }
            contributed = offer(found->second, problem, constraints, walk) || contributed;
        }
        return contributed;
    }

    // Returns whether record i joined the selection.
    bool offer(std::size_t i, const Problem& problem, const Constraints& constraints, Walk& walk) const {
        if (walk.offered[i]) { return false; }
        walk.offered[i]    = true;
        const Record& item = records_[i];
        if (!isPrimitiveAllowed(item->getName(), getEnabledPrimitives(), getDisabledPrimitives())) { return false; }
        const Result verdict = item->isApplicable(problem, constraints);
        if (!verdict.isSuccess()) {
            if (!walk.rejections.empty()) { walk.rejections += "; "; }
            walk.rejections += item->getName();
            walk.rejections += ": ";
            walk.rejections += verdict.getMessage();
            return false;
        }
        walk.chosen.push_back(i);
        return true;
    }

    std::vector<std::unique_ptr<PrimitiveBase>> instantiate(const std::vector<std::size_t>& positions,
                                                            const Problem& problem) const {
        std::vector<std::unique_ptr<PrimitiveBase>> primitives;
        primitives.reserve(positions.size());
        for (const std::size_t position : positions) {
            std::unique_ptr<PrimitiveBase> copy = records_[position]->clone();
            if (copy == nullptr) {
                throw Exception(FTRAIN_STATUS_INTERNAL_ERROR, "Applicable Primitive returned a null clone");
            }
            static_cast<Primitive<Problem>&>(*copy).configure(problem);
            primitives.push_back(std::move(copy));
        }
        return primitives;
    }

    std::vector<Record> records_;
    std::unordered_map<std::string, std::size_t> position_of_;
    mutable MemoryPrimitiveCache cache_;
};

// Every engine the library ships; the process registry registers exactly this
// list, once.
std::vector<std::shared_ptr<OpsEngineBase>> makeBuiltinOpsEngines();

}  // namespace ftrain

#endif
