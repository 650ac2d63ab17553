// C functions with the names and signatures of the reference's C API for this path
// (include/vsag/vsag_c_api.h:36-160, src/vsag_c_api.cpp): factory, destroy, build, add, train,
// knn_search.  They sit on the vsag::Factory / Index mirror, so a program written against the
// reference's C API links against libvsag_b200.so unchanged for "ivf" and "brute_force".
// vsag_index_knn_search_batch is an addition: the reference's C API takes one query per call.
// vsag_serialize_file / vsag_deserialize_file follow include/vsag/vsag_c_api.h:319-330.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <functional>

#include "vsag_host.h"

#define VSAG_C_EXPORT extern "C" __attribute__((visibility("default")))

extern "C" {
typedef struct Error {
    int code;
    char message[1024];
} Error_t;

typedef void* vsag_index_t;

typedef bool (*FilterFunc_t)(int64_t id);   // true = the id may be returned (Filter::CheckValid)

typedef struct SearchResult {
    float* dists;
    int64_t* ids;
    int64_t count;
    void* other_result;
} SearchResult_t;
}

namespace {

struct IndexBox {
    std::shared_ptr<vsag::Index> index;
};

Error_t
success() {
    Error_t e;
    e.code = 0;
    snprintf(e.message, sizeof(e.message), "%s", "success");
    return e;
}

Error_t
make_error(int code, const std::string& message) {
    Error_t e;
    e.code = code;
    snprintf(e.message, sizeof(e.message), "%s", message.c_str());
    return e;
}

Error_t
make_error(const vsag::Error& err) {
    return make_error(-static_cast<int>(err.type), err.message);  // VSAG_* codes are the negated enum
}

thread_local std::string tl_factory_error;

vsag::DatasetPtr
borrow(const float* data, const int64_t* ids, uint64_t dim, uint64_t count) {
    return vsag::Dataset::Make()
        ->Owner(false)
        ->Dim(static_cast<int64_t>(dim))
        ->NumElements(static_cast<int64_t>(count))
        ->Ids(ids)
        ->Float32Vectors(data);
}

}  // namespace

VSAG_C_EXPORT vsag_index_t
vsag_index_factory(const char* index_name, const char* index_param) {
    if (index_name == nullptr || index_param == nullptr) {
        tl_factory_error = "index name or parameter is NULL";
        return nullptr;
    }
    auto created = vsag::Factory::CreateIndex(index_name, index_param);
    if (!created.has_value()) {
        tl_factory_error = created.error().message;
        return nullptr;
    }
    return new IndexBox{created.value()};
}

// Text of the last vsag_index_factory failure on this thread (the reference logs it instead).
VSAG_C_EXPORT const char*
vsag_index_factory_error(void) {
    return tl_factory_error.c_str();
}

VSAG_C_EXPORT Error_t
vsag_index_destroy(vsag_index_t index) {
    delete static_cast<IndexBox*>(index);
    return success();
}

VSAG_C_EXPORT Error_t
vsag_index_build(vsag_index_t index, const float* data, const int64_t* ids, uint64_t dim, uint64_t count) {
    auto* box = static_cast<IndexBox*>(index);
    if (box == nullptr) {
        return make_error(-1, "index is NULL");
    }
    auto r = box->index->Build(borrow(data, ids, dim, count));
    return r.has_value() ? success() : make_error(r.error());
}

VSAG_C_EXPORT Error_t
vsag_index_add(vsag_index_t index, const float* data, const int64_t* ids, const uint64_t dim,
               const uint64_t count) {
    auto* box = static_cast<IndexBox*>(index);
    if (box == nullptr) {
        return make_error(-1, "index is NULL");
    }
    auto r = box->index->Add(borrow(data, ids, dim, count));
    return r.has_value() ? success() : make_error(r.error());
}

VSAG_C_EXPORT Error_t
vsag_index_train(vsag_index_t index, const float* data, const int64_t* ids, const uint64_t dim,
                 const uint64_t count) {
    auto* box = static_cast<IndexBox*>(index);
    if (box == nullptr) {
        return make_error(-1, "index is NULL");
    }
    auto r = box->index->Train(borrow(data, ids, dim, count));
    return r.has_value() ? success() : make_error(r.error());
}

VSAG_C_EXPORT Error_t
vsag_index_knn_search(vsag_index_t index, const float* query, uint64_t dim, int64_t k, const char* parameters,
                      SearchResult_t* search_result) {
    if (search_result == nullptr) {
        return make_error(-1, "search result is NULL");
    }
    auto* box = static_cast<IndexBox*>(index);
    if (box == nullptr) {
        return make_error(-1, "index is NULL");
    }
    if (k <= 0) {
        return make_error(-3, "knn_search requires k >= 1");
    }
    auto r = box->index->KnnSearch(borrow(query, nullptr, dim, 1), k, parameters == nullptr ? "{}" : parameters);
    if (!r.has_value()) {
        return make_error(r.error());
    }
    int64_t to_write = std::min<int64_t>(r.value()->GetDim(), k);
    for (int64_t i = 0; i < to_write; ++i) {
        search_result->ids[i] = r.value()->GetIds()[i];
        search_result->dists[i] = r.value()->GetDistances()[i];
    }
    search_result->count = to_write;
    return success();
}

// nq queries in one call: ids[nq x k], dists[nq x k], padded with -1 / +inf.
VSAG_C_EXPORT Error_t
vsag_index_knn_search_batch(vsag_index_t index, const float* queries, uint64_t dim, uint64_t nq, int64_t k,
                            const char* parameters, int64_t* ids, float* dists) {
    auto* box = static_cast<IndexBox*>(index);
    if (box == nullptr) {
        return make_error(-1, "index is NULL");
    }
    if (ids == nullptr || dists == nullptr) {
        return make_error(-3, "output buffers are NULL");
    }
    auto r = box->index->KnnSearch(borrow(queries, nullptr, dim, nq), k, parameters == nullptr ? "{}" : parameters);
    if (!r.has_value()) {
        return make_error(r.error());
    }
    const auto& res = r.value();
    for (uint64_t q = 0; q < nq; ++q) {
        for (int64_t i = 0; i < k; ++i) {
            bool have = static_cast<int64_t>(q) < res->GetNumElements() && i < res->GetDim() && res->GetIds() != nullptr;
            ids[q * k + i] = have ? res->GetIds()[q * res->GetDim() + i] : -1;
            dists[q * k + i] = have ? res->GetDistances()[q * res->GetDim() + i] : __builtin_inff();
        }
    }
    return success();
}

// Index::SearchWithRequest (include/vsag/index.h:333) for nq queries with explicit bucket lists, an addition
// to the reference's C interface: bucket_ids holds the lists of all queries back to back, bucket_counts[q]
// says how many belong to query q (bucket_counts NULL = default routing).  KNN only; ids[nq x k], dists[nq x k],
// padded with -1 / +inf.  The lists are validated as IVF::SearchWithRequest validates
// SearchRequest::bucket_ids_ (src/algorithm/ivf/ivf.cpp:2075-2112).
VSAG_C_EXPORT Error_t
vsag_index_search_with_request(vsag_index_t index, const float* queries, uint64_t dim, uint64_t nq, int64_t k,
                               const char* parameters, const int64_t* bucket_ids, const uint64_t* bucket_counts,
                               int64_t* ids, float* dists) {
    auto* box = static_cast<IndexBox*>(index);
    if (box == nullptr) {
        return make_error(-1, "index is NULL");
    }
    if (ids == nullptr || dists == nullptr) {
        return make_error(-3, "output buffers are NULL");
    }
    vsag::SearchRequest request;
    request.query_ = borrow(queries, nullptr, dim, nq);
    request.topk_ = k;
    request.params_str_ = parameters == nullptr ? "{}" : parameters;
    if (bucket_counts != nullptr) {
        uint64_t at = 0;
        request.bucket_ids_.resize(nq);
        for (uint64_t q = 0; q < nq; ++q) {
            if (bucket_counts[q] > 0) {
                if (bucket_ids == nullptr) {
                    return make_error(-3, "bucket_ids is NULL although bucket_counts names buckets");
                }
                request.bucket_ids_[q].assign(bucket_ids + at, bucket_ids + at + bucket_counts[q]);
            }
            at += bucket_counts[q];
        }
    }
    auto r = box->index->SearchWithRequest(request);
    if (!r.has_value()) {
        return make_error(r.error());
    }
    const auto& res = r.value();
    for (uint64_t q = 0; q < nq; ++q) {
        for (int64_t i = 0; i < k; ++i) {
            bool have = static_cast<int64_t>(q) < res->GetNumElements() && i < res->GetDim() && res->GetIds() != nullptr;
            ids[q * k + i] = have ? res->GetIds()[q * res->GetDim() + i] : -1;
            dists[q * k + i] = have ? res->GetDistances()[q * res->GetDim() + i] : __builtin_inff();
        }
    }
    return success();
}

// Two additions to the reference's C interface (include/vsag/vsag_c_api.h has no filter or remove
// entry point; the C++ interface does, include/vsag/index.h:186-200, 276-303).
// invalid_bits: n_words 64-bit words, bit (id & 0xFFFFFFFF) set = filtered out; may be NULL.
// deny_modulus > 0 additionally filters, through the callback overload, every id with
// id % deny_modulus == 0 (a stand-in for a host callback, for bindings that cannot pass one).
VSAG_C_EXPORT Error_t
vsag_index_knn_search_filtered(vsag_index_t index, const float* query, uint64_t dim, int64_t k, const char* parameters,
                               const uint64_t* invalid_bits, uint64_t n_words, int64_t deny_modulus,
                               SearchResult_t* search_result) {
    if (search_result == nullptr) {
        return make_error(-1, "search result is NULL");
    }
    auto* box = static_cast<IndexBox*>(index);
    if (box == nullptr) {
        return make_error(-1, "index is NULL");
    }
    if (k <= 0) {
        return make_error(-3, "knn_search requires k >= 1");
    }
    const std::string params = parameters == nullptr ? "{}" : parameters;
    auto q = borrow(query, nullptr, dim, 1);
    auto r = [&]() {
        if (deny_modulus > 0) {
            return box->index->KnnSearch(q, k, params, [=](int64_t id) { return id % deny_modulus == 0; });
        }
        auto bits = vsag::Bitset::Make();
        for (uint64_t w = 0; invalid_bits != nullptr && w < n_words; ++w) {
            for (int b = 0; b < 64; ++b) {
                if ((invalid_bits[w] >> b) & 1u) {
                    bits->Set(static_cast<int64_t>(w * 64 + b));
                }
            }
        }
        return box->index->KnnSearch(q, k, params, bits);
    }();
    if (!r.has_value()) {
        return make_error(r.error());
    }
    int64_t to_write = std::min<int64_t>(r.value()->GetDim(), k);
    for (int64_t i = 0; i < to_write; ++i) {
        search_result->ids[i] = r.value()->GetIds()[i];
        search_result->dists[i] = r.value()->GetDistances()[i];
    }
    search_result->count = to_write;
    return success();
}

VSAG_C_EXPORT Error_t
vsag_index_remove(vsag_index_t index, const int64_t* ids, uint64_t count, uint32_t* removed) {
    auto* box = static_cast<IndexBox*>(index);
    if (box == nullptr) {
        return make_error(-1, "index is NULL");
    }
    auto r = box->index->Remove(std::vector<int64_t>(ids, ids + count));
    if (!r.has_value()) {
        return make_error(r.error());
    }
    if (removed != nullptr) {
        *removed = r.value();
    }
    return success();
}

VSAG_C_EXPORT int64_t
vsag_index_get_num_elements(vsag_index_t index) {
    auto* box = static_cast<IndexBox*>(index);
    return box == nullptr ? 0 : box->index->GetNumElements();
}

VSAG_C_EXPORT Error_t
vsag_serialize_file(vsag_index_t index, const char* file_path) {
    auto* box = static_cast<IndexBox*>(index);
    if (box == nullptr) {
        return make_error(-1, "index is NULL");
    }
    if (file_path == nullptr) {
        return make_error(-static_cast<int>(vsag::ErrorType::INVALID_ARGUMENT), "file_path is NULL");
    }
    std::ofstream file(file_path, std::ios::binary);
    if (!file.is_open()) {
        return make_error(-1, "failed to open file for writing: " + std::string(file_path));
    }
    auto r = box->index->Serialize(file);
    if (!r.has_value()) {
        return make_error(r.error());
    }
    file.close();
    if (!file) {
        return make_error(-static_cast<int>(vsag::ErrorType::INTERNAL_ERROR),
                          "failed to write file: " + std::string(file_path));
    }
    return success();
}

VSAG_C_EXPORT Error_t
vsag_deserialize_file(vsag_index_t index, const char* file_path) {
    auto* box = static_cast<IndexBox*>(index);
    if (box == nullptr) {
        return make_error(-1, "index is NULL");
    }
    if (file_path == nullptr) {
        return make_error(-static_cast<int>(vsag::ErrorType::INVALID_ARGUMENT), "file_path is NULL");
    }
    std::ifstream file(file_path, std::ios::binary);
    if (!file.is_open()) {
        return make_error(-static_cast<int>(vsag::ErrorType::MISSING_FILE),
                          "failed to open file for reading: " + std::string(file_path));
    }
    auto r = box->index->Deserialize(file);
    if (!r.has_value()) {
        return make_error(r.error());
    }
    return success();
}

// include/vsag/vsag_c_api.h:174-193: k is the largest number of results (at least 1).  Addition: a
// negative k asks for every vector within the radius, as Index::RangeSearch does with a negative
// limited_size; the result arrays then need room for 512 entries (more in-radius vectors are an error).
VSAG_C_EXPORT Error_t
vsag_index_range_search(vsag_index_t index, const float* query, uint64_t dim, float radius, int64_t k,
                        const char* parameters, SearchResult_t* search_result) {
    auto* box = static_cast<IndexBox*>(index);
    if (box == nullptr) {
        return make_error(-1, "index is NULL");
    }
    if (query == nullptr || search_result == nullptr || search_result->ids == nullptr ||
        search_result->dists == nullptr) {
        return make_error(-static_cast<int>(vsag::ErrorType::INVALID_ARGUMENT), "query or search_result is NULL");
    }
    if (k == 0) {
        return make_error(-static_cast<int>(vsag::ErrorType::INVALID_ARGUMENT), "k must not be 0");
    }
    auto q = borrow(query, nullptr, dim, 1);
    auto r = box->index->RangeSearch(q, radius, parameters == nullptr ? "" : parameters, k);
    if (!r.has_value()) {
        return make_error(r.error());
    }
    const int64_t to_write = k > 0 ? std::min<int64_t>(r.value()->GetDim(), k) : r.value()->GetDim();
    for (int64_t i = 0; i < to_write; ++i) {
        search_result->ids[i] = r.value()->GetIds()[i];
        search_result->dists[i] = r.value()->GetDistances()[i];
    }
    search_result->count = to_write;
    return success();
}

namespace {

Error_t
write_result(const vsag::Expected<vsag::DatasetPtr>& r, int64_t k, SearchResult_t* search_result) {
    if (!r.has_value()) {
        return make_error(r.error());
    }
    const int64_t to_write = std::min<int64_t>(r.value()->GetDim(), k);
    for (int64_t i = 0; i < to_write; ++i) {
        search_result->ids[i] = r.value()->GetIds()[i];
        search_result->dists[i] = r.value()->GetDistances()[i];
    }
    search_result->count = to_write;
    return success();
}

}  // namespace

// include/vsag/vsag_c_api.h:152-172 and :195-216: `filter` says which ids are valid.
VSAG_C_EXPORT Error_t
vsag_index_knn_search_with_filter(vsag_index_t index, const float* query, uint64_t dim, int64_t k,
                                  const char* parameters, FilterFunc_t filter, SearchResult_t* search_result) {
    auto* box = static_cast<IndexBox*>(index);
    if (search_result == nullptr) {
        return make_error(-1, "search result is NULL");
    }
    if (box == nullptr) {
        return make_error(-1, "index is NULL");
    }
    if (k <= 0) {
        return make_error(-3, "knn_search requires k >= 1");
    }
    auto q = borrow(query, nullptr, dim, 1);
    std::function<bool(int64_t)> out;
    if (filter != nullptr) {
        out = [filter](int64_t id) { return !filter(id); };
    }
    return write_result(box->index->KnnSearch(q, k, parameters == nullptr ? "{}" : parameters, out), k, search_result);
}

VSAG_C_EXPORT Error_t
vsag_index_range_search_with_filter(vsag_index_t index, const float* query, uint64_t dim, float radius, int64_t k,
                                    const char* parameters, FilterFunc_t filter, SearchResult_t* search_result) {
    auto* box = static_cast<IndexBox*>(index);
    if (search_result == nullptr) {
        return make_error(-1, "search result is NULL");
    }
    if (box == nullptr) {
        return make_error(-1, "index is NULL");
    }
    if (k <= 0) {
        return make_error(-3, "range_search requires k >= 1 as result cap");
    }
    auto q = borrow(query, nullptr, dim, 1);
    std::function<bool(int64_t)> out;
    if (filter != nullptr) {
        out = [filter](int64_t id) { return !filter(id); };
    }
    return write_result(box->index->RangeSearch(q, radius, parameters == nullptr ? "{}" : parameters, out, k), k,
                        search_result);
}
