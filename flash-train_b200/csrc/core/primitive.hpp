// Primitive: one operator implementation, and the resources one dispatch uses.
//
// Contract as in the reference (src/include/flash_train/primitive.hpp:24-76,
// src/primitive.cpp:12-25, src/include/flash_train/resources.hpp:17-36): engines
// hold shared prototypes; creating a Plan clones a prototype and configures the
// clone for one problem; execute() enforces the workspace requirement and then
// enqueues asynchronous work.
#ifndef FTRAIN_CORE_PRIMITIVE_HPP_
#define FTRAIN_CORE_PRIMITIVE_HPP_

#include <cstdint>
#include <memory>

#include "core/constraints.hpp"
#include "core/error.hpp"

namespace ftrain {

class Resources final {
  public:
    Resources(void* workspace, std::uint64_t workspace_bytes, FTrainStream stream) noexcept
        : workspace_(workspace), workspace_bytes_(workspace_bytes), stream_(stream) {}
    void* getWorkspace() const noexcept { return workspace_; }
    std::uint64_t getWorkspaceBytes() const noexcept { return workspace_bytes_; }
    FTrainStream getStream() const noexcept { return stream_; }

  private:
    void* workspace_;
    std::uint64_t workspace_bytes_;
    FTrainStream stream_;
};

struct PrimitiveBase {
    virtual ~PrimitiveBase();

    // Stable for the object's lifetime; the identity used in diagnostics and by
    // FTRAIN_ENABLED_PRIMITIVES / FTRAIN_DISABLED_PRIMITIVES.
    virtual const char* getName() const noexcept = 0;
    virtual std::unique_ptr<PrimitiveBase> clone() const = 0;
    // Meaningful after configure().
    virtual std::uint64_t getRequiredWorkspaceBytes() const noexcept = 0;

    // Throws Exception(FTRAIN_STATUS_INVALID_ARGUMENT), without dispatching,
    // when the workspace is smaller than required or null while required.
    void execute(const Resources& resources);

  protected:
    PrimitiveBase() noexcept                       = default;
    PrimitiveBase(const PrimitiveBase&)            = default;
    PrimitiveBase& operator=(const PrimitiveBase&) = default;

    virtual void executeImpl(const Resources& resources) = 0;
};

template<typename Problem>
struct Primitive : PrimitiveBase {
    // Success, or FTRAIN_STATUS_UNSUPPORTED with the reason. Called
    // concurrently on the shared prototype.
    virtual Result isApplicable(const Problem& problem, const Constraints& constraints) const = 0;
    // Captures everything execution needs; the problem may die afterwards.
    virtual void configure(const Problem& problem) = 0;
};

}  // namespace ftrain

#endif
