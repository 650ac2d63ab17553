// Host-side mirror of the part of VSAG's public API that the accelerated path sits behind:
// vsag::Factory::CreateIndex("ivf" | "brute_force", json), Index::{Build, Train, Add, KnnSearch,
// RangeSearch, Remove, Serialize, Deserialize, GetNumElements, GetMemoryUsage} and the Dataset builder (reference: include/vsag/factory.h:47-50,
// include/vsag/index.h:126-303, include/vsag/dataset.h:135-511, include/vsag/errors.h:26-48).
// Same names, argument meaning and error behaviour, written from scratch over the C ABI of
// include/vsag_b200.h; no exception crosses these calls.
#pragma once

#include <cstdint>
#include <functional>
#include <iosfwd>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace vsag {

enum class ErrorType {
    UNKNOWN_ERROR = 1,
    INTERNAL_ERROR,
    INVALID_ARGUMENT,
    WRONG_STATUS,
    BUILD_TWICE,
    INDEX_NOT_EMPTY,
    UNSUPPORTED_INDEX,
    UNSUPPORTED_INDEX_OPERATION,
    DIMENSION_NOT_EQUAL,
    INDEX_EMPTY,
    NO_ENOUGH_MEMORY,
    READ_ERROR,
    MISSING_FILE,
    INVALID_BINARY,
};

struct Error {
    ErrorType type;
    std::string message;
};

// Stand-in for tl::expected<T, Error> with the members the API's callers use.
template <typename T>
class Expected {
public:
    Expected(T value) : has_(true), value_(std::move(value)) {}  // NOLINT(google-explicit-constructor)
    Expected(Error error) : has_(false), error_(std::move(error)) {}  // NOLINT(google-explicit-constructor)
    bool has_value() const { return has_; }
    explicit operator bool() const { return has_; }
    T& value() { return value_; }
    const T& value() const { return value_; }
    T& operator*() { return value_; }
    T* operator->() { return &value_; }
    const Error& error() const { return error_; }

private:
    bool has_;
    T value_{};
    Error error_{ErrorType::UNKNOWN_ERROR, ""};
};

// tl::expected<void, Error>: success carries no value.
template <>
class Expected<void> {
public:
    Expected() = default;
    Expected(Error error) : has_(false), error_(std::move(error)) {}  // NOLINT(google-explicit-constructor)
    bool has_value() const { return has_; }
    explicit operator bool() const { return has_; }
    const Error& error() const { return error_; }

private:
    bool has_ = true;
    Error error_{ErrorType::UNKNOWN_ERROR, ""};
};

class Dataset;
using DatasetPtr = std::shared_ptr<Dataset>;

// Builder-style container of vectors / ids / distances (include/vsag/dataset.h).  With
// Owner(true) (the default) the dataset frees ids, distances and vectors with delete[].
class Dataset : public std::enable_shared_from_this<Dataset> {
public:
    static DatasetPtr Make();
    ~Dataset();

    DatasetPtr Owner(bool is_owner);
    DatasetPtr NumElements(int64_t num_elements);
    DatasetPtr Dim(int64_t dim);
    DatasetPtr Ids(const int64_t* ids);
    DatasetPtr Distances(const float* dists);
    DatasetPtr Float32Vectors(const float* vectors);
    DatasetPtr Float16Vectors(const uint16_t* vectors);  // bf16 bit patterns for a bf16 BruteForce index
    DatasetPtr Statistics(const std::string& stats);

    int64_t GetNumElements() const { return num_elements_; }
    int64_t GetDim() const { return dim_; }
    const int64_t* GetIds() const { return ids_; }
    const float* GetDistances() const { return distances_; }
    const float* GetFloat32Vectors() const { return vectors_; }
    const uint16_t* GetFloat16Vectors() const { return half_vectors_; }
    const std::string& GetStatistics() const { return statistics_; }

private:
    Dataset() = default;
    bool owner_ = true;
    int64_t num_elements_ = 0;
    int64_t dim_ = 0;
    const int64_t* ids_ = nullptr;
    const float* distances_ = nullptr;
    const float* vectors_ = nullptr;
    const uint16_t* half_vectors_ = nullptr;
    std::string statistics_;
};

// Growable bit set for the pre-filter of a search (include/vsag/bitset.h): bit i set means that the
// vector whose id is i (id & 0xFFFFFFFF) is filtered out.
class Bitset {
public:
    static std::shared_ptr<Bitset> Make() { return std::make_shared<Bitset>(); }
    void Set(int64_t pos, bool value = true) {
        const size_t word = static_cast<size_t>(pos) >> 6;
        if (word >= words_.size()) {
            if (!value) {
                return;
            }
            words_.resize(word + 1, 0);
        }
        const uint64_t bit = uint64_t{1} << (pos & 63);
        words_[word] = value ? (words_[word] | bit) : (words_[word] & ~bit);
    }
    bool Test(int64_t pos) const {
        const size_t word = static_cast<size_t>(pos) >> 6;
        return word < words_.size() && ((words_[word] >> (pos & 63)) & 1u) != 0;
    }
    const std::vector<uint64_t>& Words() const { return words_; }

private:
    std::vector<uint64_t> words_;
};
using BitsetPtr = std::shared_ptr<Bitset>;

enum class SearchMode {
    KNN_SEARCH = 1,
    RANGE_SEARCH = 2,
};

// The request form of a search (include/vsag/search_request.h:48-227), with the fields this path
// honours; names and defaults are the reference's.  `filter_` stands for the reference's FilterPtr:
// it returns true for an id that may be returned (Filter::CheckValid).
class SearchRequest {
public:
    DatasetPtr query_{nullptr};
    SearchMode mode_{SearchMode::KNN_SEARCH};
    int64_t topk_{10};
    float radius_{0.5F};
    int64_t limited_size_{-1};
    std::string params_str_{};
    bool enable_filter_{false};
    std::function<bool(int64_t)> filter_{nullptr};
    bool enable_bitset_filter_{false};
    BitsetPtr bitset_filter_{nullptr};
    // IVF only: per query, the buckets to scan instead of routing (one list per query; empty outer
    // vector = default routing).  Validated as IVF::SearchWithRequest does
    // (src/algorithm/ivf/ivf.cpp:2075-2112).
    std::vector<std::vector<int64_t>> bucket_ids_{};
};

class Index {
public:
    virtual ~Index() = default;

    // Train + Add; returns the ids that failed to insert (always empty here).
    virtual Expected<std::vector<int64_t>> Build(const DatasetPtr& base) = 0;
    virtual Expected<void*> Train(const DatasetPtr& data) = 0;
    virtual Expected<std::vector<int64_t>> Add(const DatasetPtr& base) = 0;
    // query: NumElements >= 1 rows.  One query returns NumElements = 1, Dim = results found
    // (<= k); a batch returns NumElements = Q, Dim = k padded with id -1 / distance +inf.
    virtual Expected<DatasetPtr> KnnSearch(const DatasetPtr& query, int64_t k,
                                           const std::string& parameters) const = 0;
    // The same search with a pre-filter (include/vsag/index.h:276-303): `invalid` marks ids that are
    // filtered out; `filter` returns true for an id that is filtered out.
    virtual Expected<DatasetPtr> KnnSearch(const DatasetPtr& query, int64_t k, const std::string& parameters,
                                           BitsetPtr invalid) const = 0;
    virtual Expected<DatasetPtr> KnnSearch(const DatasetPtr& query, int64_t k, const std::string& parameters,
                                           const std::function<bool(int64_t)>& filter) const = 0;
    // Every vector within `radius` of the one query, nearest first; limited_size >= 1 keeps the nearest
    // limited_size of them, a negative one keeps all, 0 is an error (include/vsag/index.h:380-397).
    // NumElements = 1, Dim = results found.
    virtual Expected<DatasetPtr> RangeSearch(const DatasetPtr& query, float radius, const std::string& parameters,
                                             int64_t limited_size = -1) const = 0;
    // The same with a pre-filter, as for KnnSearch (include/vsag/index.h:399-441).
    virtual Expected<DatasetPtr> RangeSearch(const DatasetPtr& query, float radius, const std::string& parameters,
                                             BitsetPtr invalid, int64_t limited_size = -1) const = 0;
    virtual Expected<DatasetPtr> RangeSearch(const DatasetPtr& query, float radius, const std::string& parameters,
                                             const std::function<bool(int64_t)>& filter,
                                             int64_t limited_size = -1) const = 0;
    // Search described by a request object (include/vsag/index.h:333): KNN for one query or a batch, range
    // search for one query, optional id filter, and for IVF the explicit bucket lists of
    // SearchRequest::bucket_ids_.
    virtual Expected<DatasetPtr> SearchWithRequest(const SearchRequest& request) const = 0;
    // RemoveMode::MARK_REMOVE (include/vsag/index.h:186-200): the vectors stay stored but are never
    // returned again; the result is the number of ids found and newly marked.
    virtual Expected<uint32_t> Remove(const std::vector<int64_t>& ids) = 0;
    // Serialize to / Deserialize from an opened stream (include/vsag/index.h:903-940).  Deserialize wants
    // an empty index created with the parameters of the one that was written (INDEX_NOT_EMPTY,
    // INVALID_ARGUMENT otherwise); a stream that is not such a file gives INVALID_BINARY, a short one
    // READ_ERROR.  The bytes are this engine's own container around the pieces IVF::Serialize and
    // BruteForce::Serialize write (centroids, quantizer model, per-list codes and inner ids, labels,
    // reorder rows; src/algorithm/ivf/ivf.cpp:990-1056, src/algorithm/bruteforce/bruteforce.cpp:685-705):
    // codes are stored and reloaded verbatim, so a reloaded index answers bit for bit like the original.
    virtual Expected<void> Serialize(std::ostream& out) const = 0;
    virtual Expected<void> Deserialize(std::istream& in) = 0;
    virtual int64_t GetNumElements() const = 0;
    virtual int64_t GetMemoryUsage() const = 0;
    virtual std::string GetIndexType() const = 0;
};

class Factory {
public:
    // name: "ivf" or "brute_force" (case-insensitive).  parameters: the reference's creation JSON
    // (dtype, metric_type, dim, index_param{...}).  Unknown names -> UNSUPPORTED_INDEX, bad or
    // unknown keys / values -> INVALID_ARGUMENT.
    static Expected<std::shared_ptr<Index>> CreateIndex(const std::string& name, const std::string& parameters);
};

}  // namespace vsag
