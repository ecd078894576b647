// Result / Exception, StorageView and the argument value types.
// Behaviours pinned by the reference's tests/error_test.cpp:35-199,
// tests/storage_view_test.cpp:30-251 and tests/tensor_test.cpp.
#include <cstring>
#include <string>

#include "core/tensor.hpp"
#include "mini_test.hpp"

using namespace ftrain;

namespace {

FTrainStorageView view(void* memory, const std::int64_t* dims, std::uint8_t rank, const std::int64_t* strides = nullptr,
                       FTrainNumericType type = FTRAIN_NUMERIC_TYPE_FP32,
                       FTrainIndexType index = FTRAIN_INDEX_TYPE_CONTINUOUS, bool host = false) {
    return FTrainStorageView{memory, dims, strides, rank, type, index, host};
}

}  // namespace

TEST(result_defaults_and_plain_text) {
    Result fresh;
    CHECK(fresh.isSuccess());
    CHECK_EQ(std::string(fresh.getMessage()), std::string(""));
    Result failed(FTRAIN_STATUS_UNSUPPORTED, "50% of %s");
    CHECK_EQ(static_cast<int>(failed.getStatus()), static_cast<int>(FTRAIN_STATUS_UNSUPPORTED));
    CHECK_EQ(std::string(failed.getMessage()), std::string("50% of %s"));  // '%' is literal
    Result success(FTRAIN_STATUS_SUCCESS, "ignored");
    CHECK_EQ(std::string(success.getMessage()), std::string(""));
    Result null_text(FTRAIN_STATUS_OVERFLOW, nullptr);
    CHECK_EQ(std::string(null_text.getMessage()), std::string(""));
    failed.clear();
    CHECK(failed.isSuccess());
}

TEST(result_truncates_at_2047_characters) {
    const std::string long_text(5000, 'x');
    Result plain(FTRAIN_STATUS_INTERNAL_ERROR, long_text.c_str());
    CHECK_EQ(std::strlen(plain.getMessage()), static_cast<std::size_t>(2047));
    Result formatted;
    formatted.setFormat(FTRAIN_STATUS_INTERNAL_ERROR, "%s|%d", long_text.c_str(), 7);
    CHECK_EQ(std::strlen(formatted.getMessage()), static_cast<std::size_t>(2047));
    formatted.setFormat(FTRAIN_STATUS_INVALID_ARGUMENT, "value %d and %s", 42, "text");
    CHECK_EQ(std::string(formatted.getMessage()), std::string("value 42 and text"));
    formatted.setFormat(FTRAIN_STATUS_SUCCESS, "dropped %d", 1);
    CHECK_EQ(std::string(formatted.getMessage()), std::string(""));
    Result copy = plain;
    CHECK_EQ(std::string(copy.getMessage()), std::string(plain.getMessage()));
}

TEST(exception_never_carries_success) {
    Exception from_status(FTRAIN_STATUS_SUCCESS, "fine");
    CHECK_EQ(static_cast<int>(from_status.getResult().getStatus()), static_cast<int>(FTRAIN_STATUS_INTERNAL_ERROR));
    CHECK(std::strstr(from_status.what(), "cannot be constructed with FTRAIN_STATUS_SUCCESS") != nullptr);
    Exception from_result{Result{}};
    CHECK_EQ(static_cast<int>(from_result.getResult().getStatus()), static_cast<int>(FTRAIN_STATUS_INTERNAL_ERROR));
    Exception formatted(FTRAIN_STATUS_OVERFLOW, "%d items", 3);
    CHECK_EQ(std::string(formatted.what()), std::string("3 items"));
}

TEST(storage_view_copies_metadata) {
    float cell = 0;
    std::int64_t dims[2]    = {3, 5};
    std::int64_t strides[2] = {1, 3};
    StorageView dense(view(&cell, dims, 2));
    StorageView strided(view(&cell, dims, 2, strides, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_INVALID));
    dims[0]    = 99;  // later changes of the caller's arrays are invisible
    strides[1] = 99;
    CHECK_EQ(dense.getDims()[0], std::int64_t{3});
    CHECK(dense.getStrides().empty());
    CHECK_EQ(strided.getStrides()[1], std::int64_t{3});
    CHECK_EQ(static_cast<int>(strided.getIndexType()), static_cast<int>(FTRAIN_INDEX_TYPE_INVALID));
    StorageView copy = strided;
    CHECK(copy.getDims() == strided.getDims());
    // Rank above the inline capacity still works.
    std::int64_t many[7] = {1, 2, 3, 4, 5, 6, 7};
    StorageView wide(view(nullptr, many, 7));
    CHECK_EQ(wide.getDims().size(), static_cast<std::size_t>(7));
    CHECK_EQ(wide.getDims()[6], std::int64_t{7});
    StorageView wide_copy = wide;
    CHECK(wide_copy.getDims() == wide.getDims());
}

TEST(storage_view_validation_rules) {
    float cell = 0;
    std::int64_t dims[2]     = {2, 2};
    std::int64_t negative[2] = {2, -1};
    std::int64_t strides[2]  = {0, -4};  // stride values are not validated
    CHECK_THROWS_STATUS(StorageView(view(&cell, dims, 2, nullptr, FTRAIN_NUMERIC_TYPE_INVALID)), FTRAIN_STATUS_INVALID_ARGUMENT);
    CHECK_THROWS_STATUS(StorageView(view(&cell, dims, 2, nullptr, FTRAIN_NUMERIC_TYPE_COUNT)), FTRAIN_STATUS_INVALID_ARGUMENT);
    CHECK_THROWS_STATUS(StorageView(view(&cell, dims, 2, nullptr, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_COUNT)),
                        FTRAIN_STATUS_INVALID_ARGUMENT);
    CHECK_THROWS_STATUS(StorageView(view(nullptr, nullptr, 0)), FTRAIN_STATUS_INVALID_ARGUMENT);  // scalar needs memory
    CHECK_THROWS_STATUS(StorageView(view(&cell, nullptr, 2)), FTRAIN_STATUS_INVALID_ARGUMENT);
    CHECK_THROWS_STATUS(StorageView(view(&cell, negative, 2)), FTRAIN_STATUS_INVALID_ARGUMENT);
    CHECK_THROWS_STATUS(StorageView(view(&cell, dims, 2, nullptr, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_INVALID)),
                        FTRAIN_STATUS_INVALID_ARGUMENT);  // no layout source
    CHECK_THROWS_STATUS(StorageView(view(&cell, dims, 2, strides)), FTRAIN_STATUS_INVALID_ARGUMENT);  // two layout sources
    StorageView odd(view(&cell, dims, 2, strides, FTRAIN_NUMERIC_TYPE_UINT1, FTRAIN_INDEX_TYPE_INVALID));
    CHECK_EQ(odd.getStrides()[1], std::int64_t{-4});
    std::int64_t empty[2] = {0, 4};
    StorageView no_rows(view(nullptr, empty, 2, nullptr, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_GROUPED_CONTINUOUS));
    CHECK_EQ(no_rows.getDims()[0], std::int64_t{0});
    StorageView scalar(view(&cell, nullptr, 0, nullptr, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_CONTINUOUS, true));
    CHECK(scalar.getDims().empty() && scalar.isHostMemory());
}

TEST(grouped_tensor_shape_rules) {
    float cell = 0;
    std::int64_t data_dims[2] = {8, 4};
    std::int64_t three[1]     = {3};
    std::int64_t four[1]      = {4};
    std::int64_t square[2]    = {3, 1};
    const auto data    = [&] { return StorageView(view(&cell, data_dims, 2)); };
    const auto vector3 = [&] { return StorageView(view(&cell, three, 1, nullptr, FTRAIN_NUMERIC_TYPE_INT64)); };
    const auto vector4 = [&] { return StorageView(view(&cell, four, 1, nullptr, FTRAIN_NUMERIC_TYPE_INT64)); };
    const auto matrix  = [&] { return StorageView(view(&cell, square, 2, nullptr, FTRAIN_NUMERIC_TYPE_INT64)); };
    GroupedTensor plain(3, data(), std::nullopt, {}, {});
    CHECK_EQ(plain.getNumGroups(), 3U);
    std::vector<StorageView> sizes;
    sizes.push_back(vector3());
    sizes.push_back(vector3());
    GroupedTensor full(3, data(), vector3(), std::move(sizes), {});
    CHECK(full.getOffsets().has_value() && full.getDimSizes().size() == 2);
    GroupedTensor none(0, data(), std::nullopt, {}, {});
    CHECK_EQ(none.getNumGroups(), 0U);
    CHECK_THROWS_STATUS(GroupedTensor(3, data(), vector4(), {}, {}), FTRAIN_STATUS_INVALID_ARGUMENT);
    CHECK_THROWS_STATUS(GroupedTensor(3, data(), matrix(), {}, {}), FTRAIN_STATUS_INVALID_ARGUMENT);
    std::vector<StorageView> one;
    one.push_back(vector3());
    CHECK_THROWS_STATUS(GroupedTensor(3, data(), std::nullopt, std::move(one), {}), FTRAIN_STATUS_INVALID_ARGUMENT);
    std::vector<StorageView> wrong;
    wrong.push_back(vector3());
    wrong.push_back(vector4());
    CHECK_THROWS_STATUS(GroupedTensor(3, data(), std::nullopt, {}, std::move(wrong)), FTRAIN_STATUS_INVALID_ARGUMENT);
}
