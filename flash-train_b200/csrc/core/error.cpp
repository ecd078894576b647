#include "core/error.hpp"

#include <cstdio>
#include <cstring>

namespace ftrain {

void Result::assign(const Result& other) noexcept {
    status_ = other.status_;
    const std::size_t used = std::strlen(other.text_);
    std::memcpy(text_, other.text_, used + 1);
}

void Result::set(FTrainStatus status, const char* message) noexcept {
    status_  = status;
    text_[0] = '\0';
    if (status == FTRAIN_STATUS_SUCCESS || message == nullptr) { return; }
    const std::size_t length = strnlen(message, kCapacity - 1);
    std::memcpy(text_, message, length);
    text_[length] = '\0';
}

void Result::setFormat(FTrainStatus status, const char* format, ...) noexcept {
    std::va_list arguments;
    va_start(arguments, format);
    setVFormat(status, format, arguments);
    va_end(arguments);
}

void Result::setVFormat(FTrainStatus status, const char* format, std::va_list arguments) noexcept {
    status_  = status;
    text_[0] = '\0';
    if (status == FTRAIN_STATUS_SUCCESS || format == nullptr) { return; }
    if (std::vsnprintf(text_, kCapacity, format, arguments) < 0) { text_[0] = '\0'; }
    text_[kCapacity - 1] = '\0';
}

void Exception::rejectSuccess() noexcept {
    if (result_.isSuccess()) {
        result_.set(FTRAIN_STATUS_INTERNAL_ERROR, "Exception cannot be constructed with FTRAIN_STATUS_SUCCESS");
    }
}

Exception::Exception(const Result& result) noexcept : result_(result) { rejectSuccess(); }

Exception::Exception(FTrainStatus status, const char* format, ...) noexcept {
    std::va_list arguments;
    va_start(arguments, format);
    result_.setVFormat(status, format, arguments);
    va_end(arguments);
    rejectSuccess();
}

}  // namespace ftrain
