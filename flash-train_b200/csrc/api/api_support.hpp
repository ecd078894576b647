// Shared plumbing of the extern "C" layer: the objects behind the opaque
// handles, the per-thread last-result slot, and the exception boundary.
// Reference: src/include/flash_train/api.hpp:36-88, src/api/common_api.cpp:9-26.
#ifndef FTRAIN_API_API_SUPPORT_HPP_
#define FTRAIN_API_API_SUPPORT_HPP_

#include <exception>
#include <new>
#include <type_traits>
#include <utility>

#include "core/error.hpp"
#include "core/ops_args.hpp"
#include "core/pattern.hpp"
#include "core/plan.hpp"

namespace ftrain {

// The calling thread's last API result: SUCCESS and "" on a fresh thread.
const Result& getLastResult() noexcept;
void clearLastResult() noexcept;
void setLastResult(FTrainStatus status, const char* message) noexcept;

// Runs `body` and converts every way it can end into a status, mirrored in the
// thread's last result: normal return -> SUCCESS; Exception -> its status and
// message; bad_alloc -> OUT_OF_MEMORY; other std::exception -> INTERNAL_ERROR
// with what(); anything else -> INTERNAL_ERROR with a fixed message.
template<typename Body>
FTrainStatus invokeApi(Body&& body) noexcept {
    static_assert(std::is_void_v<std::invoke_result_t<Body&&>>, "invokeApi body must return void");
    try {
        std::forward<Body>(body)();
        clearLastResult();
        return FTRAIN_STATUS_SUCCESS;
    } catch (const Exception& error) {
        setLastResult(error.getResult().getStatus(), error.getResult().getMessage());
        return error.getResult().getStatus();
    } catch (const std::bad_alloc& error) {
        setLastResult(FTRAIN_STATUS_OUT_OF_MEMORY, error.what());
        return FTRAIN_STATUS_OUT_OF_MEMORY;
    } catch (const std::exception& error) {
        setLastResult(FTRAIN_STATUS_INTERNAL_ERROR, error.what());
        return FTRAIN_STATUS_INTERNAL_ERROR;
    } catch (...) {
        setLastResult(FTRAIN_STATUS_INTERNAL_ERROR, "Unknown exception caught at C API boundary");
        return FTRAIN_STATUS_INTERNAL_ERROR;
    }
}

// Throws Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "<function>: <what> must not be null").
void requireNonNull(const void* pointer, const char* function, const char* what);

}  // namespace ftrain

// The structs the public opaque handle types point to.
struct FTrainPatternStruct final {
    ftrain::PatternBuilder builder;
};

struct FTrainOpsStruct final {
    explicit FTrainOpsStruct(ftrain::Ops&& value) : ops(std::move(value)) {}
    ftrain::Ops ops;
};

struct FTrainArgsStruct final {
    explicit FTrainArgsStruct(ftrain::Args&& value) : args(std::move(value)) {}
    ftrain::Args args;
};

struct FTrainPlanStruct final {
    explicit FTrainPlanStruct(ftrain::Plan&& value) : plan(std::move(value)) {}
    ftrain::Plan plan;
};

#endif
