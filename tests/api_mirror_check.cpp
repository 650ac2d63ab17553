// Compile-only check that the host layer's mirror of VSAG's public API (vsag_b200/host/vsag_host.h) stays
// source-compatible with the reference's own headers: the same generic user code is instantiated against
// namespace vsag of the reference (include/vsag/{index,dataset,factory,errors,bitset,search_request}.h) and
// against the mirror (renamed to vsag_mirror for this translation unit), and the error codes, search modes and
// request fields are compared with static_asserts.  Never linked or run: g++ -fsyntax-only.
#include <cstdint>
#include <functional>
#include <iosfwd>
#include <memory>
#include <sstream>
#include <string>
#include <type_traits>
#include <vector>

#include <vsag/bitset.h>
#include <vsag/dataset.h>
#include <vsag/errors.h>
#include <vsag/factory.h>
#include <vsag/index.h>
#include <vsag/search_request.h>

#define vsag vsag_mirror
#include "vsag_host.h"
#undef vsag

struct Reference {
    using Index = vsag::Index;
    using Dataset = vsag::Dataset;
    using DatasetPtr = vsag::DatasetPtr;
    using Bitset = vsag::Bitset;
    using BitsetPtr = vsag::BitsetPtr;
    using SearchRequest = vsag::SearchRequest;
    using SearchMode = vsag::SearchMode;
    using Error = vsag::Error;
    using ErrorType = vsag::ErrorType;
    using Factory = vsag::Factory;
};

struct Mirror {
    using Index = vsag_mirror::Index;
    using Dataset = vsag_mirror::Dataset;
    using DatasetPtr = vsag_mirror::DatasetPtr;
    using Bitset = vsag_mirror::Bitset;
    using BitsetPtr = vsag_mirror::BitsetPtr;
    using SearchRequest = vsag_mirror::SearchRequest;
    using SearchMode = vsag_mirror::SearchMode;
    using Error = vsag_mirror::Error;
    using ErrorType = vsag_mirror::ErrorType;
    using Factory = vsag_mirror::Factory;
};

// What a user of the path writes, once; it must compile against both sets of headers.
template <class V>
int64_t
user_code(const float* vectors, const int64_t* labels) {
    typename V::DatasetPtr base =
        V::Dataset::Make()->NumElements(int64_t{1})->Dim(int64_t{4})->Ids(labels)->Float32Vectors(vectors)->Owner(false);
    auto created = V::Factory::CreateIndex(std::string("ivf"), std::string("{}"));
    if (!created.has_value()) {
        typename V::ErrorType type = created.error().type;
        std::string message = created.error().message;
        return static_cast<int64_t>(type) + static_cast<int64_t>(message.size());
    }
    std::shared_ptr<typename V::Index> index = created.value();
    auto built = index->Build(base);
    std::vector<int64_t> failed_ids = built.value();
    auto trained = index->Train(base);
    auto added = index->Add(base);
    failed_ids = added.value();

    const std::string parameters = "{\"ivf\":{\"scan_buckets_count\":4}}";
    auto plain = index->KnnSearch(base, int64_t{10}, parameters);
    typename V::DatasetPtr result = plain.value();
    const int64_t* ids = result->GetIds();
    const float* distances = result->GetDistances();
    int64_t found = result->GetDim() * result->GetNumElements();
    typename V::BitsetPtr invalid = V::Bitset::Make();
    invalid->Set(int64_t{3});
    bool is_set = invalid->Test(int64_t{3});
    auto with_bitset = index->KnnSearch(base, int64_t{10}, parameters, invalid);
    std::function<bool(int64_t)> callback = [](int64_t id) { return id % 2 == 0; };
    auto with_callback = index->KnnSearch(base, int64_t{10}, parameters, callback);
    auto in_range = index->RangeSearch(base, 0.5F, parameters, int64_t{-1});
    auto in_range_default = index->RangeSearch(base, 0.5F, parameters);

    typename V::SearchRequest request;
    request.query_ = base;
    request.mode_ = V::SearchMode::KNN_SEARCH;
    request.topk_ = 5;
    request.radius_ = 0.25F;
    request.limited_size_ = -1;
    request.params_str_ = parameters;
    request.enable_bitset_filter_ = true;
    request.bitset_filter_ = invalid;
    request.bucket_ids_ = {{1, 2}};
    auto by_request = index->SearchWithRequest(request);
    typename V::DatasetPtr by_request_result = by_request.value();

    auto removed = index->Remove(std::vector<int64_t>{1});
    uint32_t removed_count = removed.value();
    std::stringstream stream;
    auto saved = index->Serialize(static_cast<std::ostream&>(stream));
    auto loaded = index->Deserialize(static_cast<std::istream&>(stream));
    bool ok = saved.has_value() && loaded.has_value() && trained.has_value() && with_bitset.has_value() &&
              with_callback.has_value() && in_range.has_value() && in_range_default.has_value() && is_set;
    return index->GetNumElements() + index->GetMemoryUsage() + found + removed_count + (ok ? 1 : 0) +
           (ids != nullptr ? 1 : 0) + (distances != nullptr ? 1 : 0) + by_request_result->GetDim();
}

template int64_t user_code<Reference>(const float*, const int64_t*);
template int64_t user_code<Mirror>(const float*, const int64_t*);

// error codes: the C ABI's status codes are the negated enumerators (include/vsag/errors.h:26-48)
#define SAME_ERROR(name)                                                                            \
    static_assert(static_cast<int>(vsag::ErrorType::name) == static_cast<int>(vsag_mirror::ErrorType::name), \
                  "ErrorType::" #name " differs from the reference")
SAME_ERROR(UNKNOWN_ERROR);
SAME_ERROR(INTERNAL_ERROR);
SAME_ERROR(INVALID_ARGUMENT);
SAME_ERROR(WRONG_STATUS);
SAME_ERROR(BUILD_TWICE);
SAME_ERROR(INDEX_NOT_EMPTY);
SAME_ERROR(UNSUPPORTED_INDEX);
SAME_ERROR(UNSUPPORTED_INDEX_OPERATION);
SAME_ERROR(DIMENSION_NOT_EQUAL);
SAME_ERROR(INDEX_EMPTY);
SAME_ERROR(NO_ENOUGH_MEMORY);
SAME_ERROR(READ_ERROR);
SAME_ERROR(MISSING_FILE);
SAME_ERROR(INVALID_BINARY);
static_assert(static_cast<int>(vsag::SearchMode::KNN_SEARCH) == static_cast<int>(vsag_mirror::SearchMode::KNN_SEARCH) &&
                  static_cast<int>(vsag::SearchMode::RANGE_SEARCH) == static_cast<int>(vsag_mirror::SearchMode::RANGE_SEARCH),
              "SearchMode differs from the reference");

// request fields this path honours: same names, same types
#define SAME_FIELD(name)                                                                                     \
    static_assert(std::is_same<decltype(vsag::SearchRequest::name), decltype(vsag_mirror::SearchRequest::name)>::value, \
                  "SearchRequest::" #name " has another type than the reference's")
SAME_FIELD(topk_);
SAME_FIELD(radius_);
SAME_FIELD(limited_size_);
SAME_FIELD(params_str_);
SAME_FIELD(enable_filter_);
SAME_FIELD(enable_bitset_filter_);
SAME_FIELD(bucket_ids_);
static_assert(std::is_same<decltype(vsag::Error::message), decltype(vsag_mirror::Error::message)>::value, "Error::message");

int
main() {
    return 0;
}
