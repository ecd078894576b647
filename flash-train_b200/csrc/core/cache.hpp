// Selection cache and the environment switches that steer selection.
//
// Observable behaviour follows the reference (src/include/flash_train/cache.hpp:27-168,
// src/cache.cpp:19-194, pinned by tests/cache/cache_test.cpp:35-234):
//   * a key is a 128-bit digest of two token groups (runtime constraints, then
//     problem description), each group prefixed by its length so that moving a
//     token across the group boundary changes the key;
//   * the first selection published for a key wins; an empty one is rejected;
//   * entries are spread over independently locked shards; a full shard evicts
//     its least-hit eighth (at least one entry) before accepting a new key;
//   * FTRAIN_ENABLED_PRIMITIVES / FTRAIN_DISABLED_PRIMITIVES /
//     FTRAIN_DISABLED_FINDERS / FTRAIN_DISABLE_CACHE are read once.
// A selection is stored as positions into the owning engine's record list.
#ifndef FTRAIN_CORE_CACHE_HPP_
#define FTRAIN_CORE_CACHE_HPP_

#include <atomic>
#include <cstddef>
#include <cstdint>
#include <memory>
#include <optional>
#include <shared_mutex>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace ftrain {

class CacheKey final {
  public:
    CacheKey(const std::vector<std::uint64_t>& constraints_tokens,
             const std::vector<std::uint64_t>& problem_tokens) noexcept;

    bool operator==(const CacheKey& other) const noexcept { return lo_ == other.lo_ && hi_ == other.hi_; }
    bool operator!=(const CacheKey& other) const noexcept { return !(*this == other); }
    std::size_t getHash() const noexcept { return static_cast<std::size_t>(lo_); }

  private:
    std::uint64_t lo_;
    std::uint64_t hi_;
};

struct CacheKeyHasher {
    std::size_t operator()(const CacheKey& key) const noexcept { return key.getHash(); }
};

class MemoryPrimitiveCache final {
  public:
    static constexpr std::size_t kDefaultMaxEntries = 30000000;
    static constexpr std::size_t kDefaultShardCount = 256;

    // A zero limit or shard count throws Exception(FTRAIN_STATUS_INVALID_ARGUMENT).
    explicit MemoryPrimitiveCache(std::size_t max_entries = kDefaultMaxEntries,
                                  std::size_t shard_count = kDefaultShardCount);

    // A hit copies the positions out under the shard lock and counts one hit.
    std::optional<std::vector<std::size_t>> find(const CacheKey& key) const;
    // Keeps an existing mapping; throws Exception(FTRAIN_STATUS_INVALID_ARGUMENT)
    // for an empty selection.
    void publish(const CacheKey& key, std::vector<std::size_t> positions);
    std::size_t getSize() const;

  private:
    struct Entry {
        std::vector<std::size_t> positions;
        mutable std::atomic<std::uint64_t> hits{0};
    };
    struct Shard {
        mutable std::shared_mutex mutex;
        // Entries are heap nodes so that rehashing never moves an atomic.
        std::unordered_map<CacheKey, std::unique_ptr<Entry>, CacheKeyHasher> entries;
        std::size_t limit{0};
    };
    Shard& shardOf(const CacheKey& key) const { return *shards_[key.getHash() % shards_.size()]; }
    static void evictColdest(Shard& shard);

    std::vector<std::unique_ptr<Shard>> shards_;
};

// Splits "a, b ,c" into {"a","b","c"}; blank entries vanish. Null -> empty.
std::unordered_set<std::string> parseNameList(const char* text);
// True when text, stripped of spaces and tabs, is neither empty nor "0".
bool parseSwitch(const char* text) noexcept;

inline bool isPrimitiveAllowed(const std::string& name, const std::unordered_set<std::string>& enabled,
                               const std::unordered_set<std::string>& disabled) {
    if (!enabled.empty() && enabled.count(name) == 0) { return false; }
    return disabled.count(name) == 0;
}

// Process-wide values, each parsed from its environment variable on first use.
const std::unordered_set<std::string>& getEnabledPrimitives();
const std::unordered_set<std::string>& getDisabledPrimitives();
const std::unordered_set<std::string>& getDisabledFinders();
bool isSelectionCacheDisabled();

inline bool isFinderDisabled(const std::string& name) { return getDisabledFinders().count(name) != 0; }

}  // namespace ftrain

#endif
