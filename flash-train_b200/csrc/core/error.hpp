// Status + message value type and the exception that carries it.
//
// Behaviour follows the reference's error model (src/include/flash_train/error.hpp:19-81,
// src/error.cpp:10-61): a Result stores a status and an inline, always
// NUL-terminated message of at most 2047 characters; a successful Result has an
// empty message; an Exception can never carry FTRAIN_STATUS_SUCCESS.
#ifndef FTRAIN_CORE_ERROR_HPP_
#define FTRAIN_CORE_ERROR_HPP_

#include <cstdarg>
#include <cstddef>
#include <exception>

#include "flash_train/common.h"

namespace ftrain {

class Result final {
  public:
    // Capacity of the inline message buffer, terminator included.
    static constexpr std::size_t kCapacity = 2048;

    Result() noexcept { text_[0] = '\0'; }
    Result(FTrainStatus status, const char* message) noexcept { set(status, message); }
    // Copies only the used part of the buffer: a Result is 2 KiB and sits on
    // paths that run per call.
    Result(const Result& other) noexcept { assign(other); }
    Result& operator=(const Result& other) noexcept {
        if (this != &other) { assign(other); }
        return *this;
    }

    void clear() noexcept {
        status_  = FTRAIN_STATUS_SUCCESS;
        text_[0] = '\0';
    }

    // Plain-text copy ('%' is literal). SUCCESS or a null message store "".
    void set(FTrainStatus status, const char* message) noexcept;
    // printf-style. SUCCESS, a null format or a formatting failure store "".
    void setFormat(FTrainStatus status, const char* format, ...) noexcept __attribute__((format(printf, 3, 4)));
    void setVFormat(FTrainStatus status, const char* format, std::va_list arguments) noexcept;

    bool isSuccess() const noexcept { return status_ == FTRAIN_STATUS_SUCCESS; }
    FTrainStatus getStatus() const noexcept { return status_; }
    const char* getMessage() const noexcept { return text_; }

  private:
    void assign(const Result& other) noexcept;

    FTrainStatus status_{FTRAIN_STATUS_SUCCESS};
    char text_[kCapacity];
};

class Exception final : public std::exception {
  public:
    explicit Exception(const Result& result) noexcept;
    Exception(FTrainStatus status, const char* format, ...) noexcept __attribute__((format(printf, 3, 4)));

    const Result& getResult() const noexcept { return result_; }
    const char* what() const noexcept override { return result_.getMessage(); }

  private:
    void rejectSuccess() noexcept;
    Result result_;
};

}  // namespace ftrain

#endif
