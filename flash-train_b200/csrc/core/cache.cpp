#include "core/cache.hpp"

#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <utility>

#include "core/error.hpp"
#include "flash_train/env.h"

namespace ftrain {
namespace {

// Two unrelated 64-bit mixers, so that a collision in one lane is independent
// of the other: lane "lo" is a multiply-rotate chain, lane "hi" a
// splitmix-style finaliser chain.
std::uint64_t rotl(std::uint64_t x, int r) noexcept { return (x << r) | (x >> (64 - r)); }

void feedLo(std::uint64_t& state, std::uint64_t token) noexcept {
    state ^= rotl(token * 0x87C37B91114253D5ULL, 31) * 0x4CF5AD432745937FULL;
    state = rotl(state, 27) * 5 + 0x52DCE729;
}

void feedHi(std::uint64_t& state, std::uint64_t token) noexcept {
    std::uint64_t z = state + 0x9E3779B97F4A7C15ULL + token;
    z               = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z               = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    state           = z ^ (z >> 31);
}

template<typename Feed>
std::uint64_t digest(std::uint64_t seed, Feed feed, const std::vector<std::uint64_t>& first,
                     const std::vector<std::uint64_t>& second) noexcept {
    std::uint64_t state = seed;
    feed(state, first.size());
    for (const std::uint64_t token : first) { feed(state, token); }
    feed(state, second.size());
    for (const std::uint64_t token : second) { feed(state, token); }
    return state;
}

std::string strip(const std::string& text) {
    const auto first = text.find_first_not_of(" \t");
    if (first == std::string::npos) { return {}; }
    const auto last = text.find_last_not_of(" \t");
    return text.substr(first, last - first + 1);
}

}  // namespace

CacheKey::CacheKey(const std::vector<std::uint64_t>& constraints_tokens,
                   const std::vector<std::uint64_t>& problem_tokens) noexcept
    : lo_(digest(0x243F6A8885A308D3ULL, feedLo, constraints_tokens, problem_tokens)),
      hi_(digest(0x13198A2E03707344ULL, feedHi, constraints_tokens, problem_tokens)) {}

MemoryPrimitiveCache::MemoryPrimitiveCache(std::size_t max_entries, std::size_t shard_count) {
    if (max_entries == 0) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "MemoryPrimitiveCache requires a positive entry limit");
    }
    if (shard_count == 0) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "MemoryPrimitiveCache requires a positive shard count");
    }
    const std::size_t share = std::max<std::size_t>(1, (max_entries + shard_count - 1) / shard_count);
    shards_.reserve(shard_count);
    for (std::size_t i = 0; i < shard_count; ++i) {
        shards_.push_back(std::make_unique<Shard>());
        shards_.back()->limit = share;
    }
}

std::optional<std::vector<std::size_t>> MemoryPrimitiveCache::find(const CacheKey& key) const {
    const Shard& shard = shardOf(key);
    const std::shared_lock<std::shared_mutex> lock(shard.mutex);
    const auto found = shard.entries.find(key);
    if (found == shard.entries.end()) { return std::nullopt; }
    found->second->hits.fetch_add(1, std::memory_order_relaxed);
    return found->second->positions;
}

void MemoryPrimitiveCache::publish(const CacheKey& key, std::vector<std::size_t> positions) {
    if (positions.empty()) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "MemoryPrimitiveCache cannot publish an empty selection");
    }
    Shard& shard = shardOf(key);
    const std::unique_lock<std::shared_mutex> lock(shard.mutex);
    if (shard.entries.find(key) != shard.entries.end()) { return; }
    if (shard.entries.size() >= shard.limit) { evictColdest(shard); }
    auto entry       = std::make_unique<Entry>();
    entry->positions = std::move(positions);
    shard.entries.emplace(key, std::move(entry));
}

void MemoryPrimitiveCache::evictColdest(Shard& shard) {
    const std::size_t batch = std::max<std::size_t>(1, shard.entries.size() / 8);
    std::vector<std::pair<std::uint64_t, CacheKey>> by_hits;
    by_hits.reserve(shard.entries.size());
    for (const auto& item : shard.entries) {
        by_hits.emplace_back(item.second->hits.load(std::memory_order_relaxed), item.first);
    }
    std::nth_element(by_hits.begin(), by_hits.begin() + static_cast<std::ptrdiff_t>(batch - 1), by_hits.end(),
                     [](const auto& a, const auto& b) { return a.first < b.first; });
    for (std::size_t i = 0; i < batch; ++i) { shard.entries.erase(by_hits[i].second); }
}

std::size_t MemoryPrimitiveCache::getSize() const {
    std::size_t total = 0;
    for (const auto& shard : shards_) {
        const std::shared_lock<std::shared_mutex> lock(shard->mutex);
        total += shard->entries.size();
    }
    return total;
}

std::unordered_set<std::string> parseNameList(const char* text) {
    std::unordered_set<std::string> names;
    if (text == nullptr) { return names; }
    const std::string all(text);
    std::size_t begin = 0;
    while (true) {
        const std::size_t comma = all.find(',', begin);
        std::string name        = strip(all.substr(begin, comma == std::string::npos ? std::string::npos : comma - begin));
        if (!name.empty()) { names.insert(std::move(name)); }
        if (comma == std::string::npos) { break; }
        begin = comma + 1;
    }
    return names;
}

bool parseSwitch(const char* text) noexcept {
    if (text == nullptr) { return false; }
    try {
        const std::string value = strip(text);
        return !value.empty() && value != "0";
    } catch (...) { return false; }
}

const std::unordered_set<std::string>& getEnabledPrimitives() {
    static const std::unordered_set<std::string> names = parseNameList(std::getenv(FTRAIN_ENABLED_PRIMITIVES));
    return names;
}

const std::unordered_set<std::string>& getDisabledPrimitives() {
    static const std::unordered_set<std::string> names = parseNameList(std::getenv(FTRAIN_DISABLED_PRIMITIVES));
    return names;
}

const std::unordered_set<std::string>& getDisabledFinders() {
    static const std::unordered_set<std::string> names = parseNameList(std::getenv(FTRAIN_DISABLED_FINDERS));
    return names;
}

bool isSelectionCacheDisabled() {
    static const bool disabled = parseSwitch(std::getenv(FTRAIN_DISABLE_CACHE));
    return disabled;
}

}  // namespace ftrain
