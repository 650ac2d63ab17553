// Implementation of the vsag::Factory / Index / Dataset mirror over the C ABI (include/vsag_b200.h).
#include "vsag_host.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <istream>
#include <limits>
#include <mutex>
#include <ostream>
#include <random>
#include <set>

#include "../../include/vsag_b200.h"
#include "json_lite.h"

namespace vsag {

using vsag_b200_host::Json;

namespace {

struct HostException {
    ErrorType type;
    std::string message;
};

[[noreturn]] void
fail(ErrorType type, const std::string& message) {
    throw HostException{type, message};
}

void
check_argument(bool cond, const std::string& message) {
    if (!cond) {
        fail(ErrorType::INVALID_ARGUMENT, message);
    }
}

// Status of a C-ABI call -> the ErrorType with the same number (codes are the negated enum values,
// as in include/vsag/vsag_c_api.h:20-34).
void
check_status(int status) {
    if (status == 0) {
        return;
    }
    char msg[1024];
    vb200_last_error(msg, sizeof(msg));
    int code = -status;
    if (code < 1 || code > static_cast<int>(ErrorType::INVALID_BINARY)) {
        code = static_cast<int>(ErrorType::UNKNOWN_ERROR);
    }
    fail(static_cast<ErrorType>(code), msg);
}

// Runs `fn`, mapping every failure to an Error the way SAFE_CALL does (src/common.h:23-35).
template <typename T, typename Fn>
Expected<T>
safe_call(Fn&& fn) {
    try {
        return Expected<T>(fn());
    } catch (const HostException& e) {
        return Expected<T>(Error{e.type, e.message});
    } catch (const std::bad_alloc&) {
        return Expected<T>(Error{ErrorType::NO_ENOUGH_MEMORY, "bad alloc"});
    } catch (const std::invalid_argument& e) {
        return Expected<T>(Error{ErrorType::INVALID_ARGUMENT, e.what()});
    } catch (const std::exception& e) {
        return Expected<T>(Error{ErrorType::UNKNOWN_ERROR, e.what()});
    }
}

// Runs `fn` for an operation without a result, mapping failures like safe_call.
template <typename Fn>
Expected<void>
safe_void(Fn&& fn) {
    auto r = safe_call<bool>([&]() {
        fn();
        return true;
    });
    if (!r.has_value()) {
        return Expected<void>(r.error());
    }
    return Expected<void>();
}

// Index file: header (magic, version, kind, creation parameters), then the blocks of the kind, then
// the end mark.  Integers and floats are little-endian, as the reference's StreamWriter writes them.
constexpr char FILE_MAGIC[8] = {'V', 'B', '2', '0', '0', 'I', 'D', 'X'};
constexpr uint32_t FILE_VERSION = 1;
constexpr uint32_t FILE_KIND_IVF = 1, FILE_KIND_BRUTE_FORCE = 2;
constexpr uint64_t FILE_END_MARK = 0x444e455f30303242ull;

template <typename T>
void
write_pod(std::ostream& out, const T& v) {
    out.write(reinterpret_cast<const char*>(&v), sizeof(T));
}

template <typename T>
void
write_array(std::ostream& out, const std::vector<T>& v) {
    write_pod<uint64_t>(out, v.size());
    out.write(reinterpret_cast<const char*>(v.data()), static_cast<std::streamsize>(v.size() * sizeof(T)));
}

template <typename T>
T
read_pod(std::istream& in) {
    T v{};
    in.read(reinterpret_cast<char*>(&v), sizeof(T));
    if (!in) {
        fail(ErrorType::READ_ERROR, "unexpected end of the index stream");
    }
    return v;
}

// An array whose length must be `want` (sizes follow from the header, so a wrong one means a damaged file).
template <typename T>
std::vector<T>
read_array(std::istream& in, uint64_t want, const char* what) {
    uint64_t n = read_pod<uint64_t>(in);
    if (n != want) {
        fail(ErrorType::INVALID_BINARY, std::string("index stream: block ") + what + " has " + std::to_string(n) +
                                            " entries, expected " + std::to_string(want));
    }
    std::vector<T> v(n);
    in.read(reinterpret_cast<char*>(v.data()), static_cast<std::streamsize>(n * sizeof(T)));
    if (!in) {
        fail(ErrorType::READ_ERROR, std::string("unexpected end of the index stream in block ") + what);
    }
    return v;
}

template <typename T>
std::vector<T>
read_array_any(std::istream& in, const char* what) {
    uint64_t n = read_pod<uint64_t>(in);
    if (n > (uint64_t{1} << 40) / sizeof(T)) {
        fail(ErrorType::INVALID_BINARY, std::string("index stream: block ") + what + " is implausibly large");
    }
    std::vector<T> v(n);
    in.read(reinterpret_cast<char*>(v.data()), static_cast<std::streamsize>(n * sizeof(T)));
    if (!in) {
        fail(ErrorType::READ_ERROR, std::string("unexpected end of the index stream in block ") + what);
    }
    return v;
}

struct FileHeader {
    uint32_t kind, dim, nlist, use_reorder;
    int32_t metric, quant;
};

void
write_header(std::ostream& out, const FileHeader& h) {
    out.write(FILE_MAGIC, sizeof(FILE_MAGIC));
    write_pod(out, FILE_VERSION);
    write_pod(out, h);
}

// Reads the header and checks it against the parameters of the index that is being filled.
void
read_header(std::istream& in, const FileHeader& want) {
    char magic[sizeof(FILE_MAGIC)] = {};
    in.read(magic, sizeof(magic));
    if (!in) {
        fail(ErrorType::READ_ERROR, "unexpected end of the index stream");
    }
    if (std::memcmp(magic, FILE_MAGIC, sizeof(magic)) != 0) {
        fail(ErrorType::INVALID_BINARY, "the stream does not hold an index written by this engine");
    }
    uint32_t version = read_pod<uint32_t>(in);
    if (version != FILE_VERSION) {
        fail(ErrorType::INVALID_BINARY, "index stream version " + std::to_string(version) + " is not supported");
    }
    FileHeader h = read_pod<FileHeader>(in);
    check_argument(h.kind == want.kind, "the stream holds another kind of index");
    check_argument(h.dim == want.dim && h.metric == want.metric && h.nlist == want.nlist && h.quant == want.quant &&
                       h.use_reorder == want.use_reorder,
                   "the index was written with other creation parameters (dim, metric_type, buckets_count, "
                   "base_quantization_type or use_reorder differ)");
}

void
check_stream_written(std::ostream& out) {
    write_pod(out, FILE_END_MARK);
    if (!out) {
        fail(ErrorType::INTERNAL_ERROR, "writing the index stream failed");
    }
}

void
check_end_mark(std::istream& in) {
    if (read_pod<uint64_t>(in) != FILE_END_MARK) {
        fail(ErrorType::INVALID_BINARY, "index stream: end mark not found");
    }
}

std::string
lower(std::string s) {
    std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return std::tolower(c); });
    return s;
}

// Keys of `obj` must all be in `allowed` (the reference rejects unknown index_param keys,
// tests/test_ivf.cpp:1148-1165).
void
check_known_keys(const Json& obj, const std::set<std::string>& allowed, const std::string& where) {
    for (const auto& m : obj.members) {
        check_argument(allowed.count(m.first) != 0, "unknown parameter \"" + m.first + "\" in " + where);
    }
}

int64_t
get_int(const Json& obj, const std::string& key, int64_t fallback) {
    const Json* v = obj.Find(key);
    if (v == nullptr) {
        return fallback;
    }
    check_argument(v->IsInteger(), "parameter \"" + key + "\" must be an integer");
    return static_cast<int64_t>(v->number);
}

bool
get_bool(const Json& obj, const std::string& key, bool fallback) {
    const Json* v = obj.Find(key);
    if (v == nullptr) {
        return fallback;
    }
    check_argument(v->IsBool(), "parameter \"" + key + "\" must be a boolean");
    return v->boolean;
}

std::string
get_string(const Json& obj, const std::string& key, const std::string& fallback) {
    const Json* v = obj.Find(key);
    if (v == nullptr) {
        return fallback;
    }
    check_argument(v->IsString(), "parameter \"" + key + "\" must be a string");
    return v->text;
}

double
get_number(const Json& obj, const std::string& key, double fallback) {
    const Json* v = obj.Find(key);
    if (v == nullptr) {
        return fallback;
    }
    check_argument(v->IsNumber(), "parameter \"" + key + "\" must be a number");
    return v->number;
}

struct CommonParam {
    uint32_t dim = 0;
    int metric = VB200_METRIC_L2;
    Json index_param;
};

// IndexCommonParam::CheckAndCreate (src/index_common_param.cpp:117-174): dtype, metric_type and dim
// are required.
CommonParam
parse_common(const std::string& parameters) {
    Json root = Json::Parse(parameters);
    check_argument(root.IsObject(), "parameters must be a JSON object");
    CommonParam out;
    check_argument(root.Contains("dtype"), "parameters must contains dtype");
    std::string dtype = get_string(root, "dtype", "");
    check_argument(dtype == "float32",
                   "parameters[dtype] must be float32 for the ivf / brute_force GPU engine, got " + dtype);
    check_argument(root.Contains("metric_type"), "parameters must contains metric_type");
    std::string metric = get_string(root, "metric_type", "");
    if (metric == "l2") {
        out.metric = VB200_METRIC_L2;
    } else if (metric == "ip") {
        out.metric = VB200_METRIC_IP;
    } else if (metric == "cosine") {
        out.metric = VB200_METRIC_COSINE;
    } else {
        fail(ErrorType::INVALID_ARGUMENT, "parameters[metric_type] must in [l2, ip, cosine], now is " + metric);
    }
    check_argument(root.Contains("dim"), "parameters must contain dim");
    const Json& dim = root.At("dim");
    check_argument(dim.IsInteger(), "parameters[dim] must be integer type");
    check_argument(dim.number > 0, "parameters[dim] must be greater than 0");
    out.dim = static_cast<uint32_t>(dim.number);
    if (root.Contains("index_param")) {
        out.index_param = root.At("index_param");
        check_argument(out.index_param.IsObject(), "parameters[index_param] must be an object");
    } else {
        out.index_param.kind = Json::Kind::Object;
    }
    return out;
}

DatasetPtr
make_empty_result() {
    // Empty index / empty query: a Dim = 0 dataset (src/index/index_impl.h:60-63, :317-320).
    return Dataset::Make()->NumElements(1)->Dim(0);
}

// Packs nq x k padded rows into a result dataset; a single query is trimmed to the entries found
// (src/utils/util_functions.cpp:68-80), a batch keeps the padding (src/algorithm/ivf/ivf.cpp:2202-2209).
DatasetPtr
pack_result(int64_t* ids, float* dists, int64_t nq, int64_t k, const std::string& stats) {
    int64_t dim = k;
    if (nq == 1) {
        dim = 0;
        while (dim < k && ids[dim] >= 0) {
            ++dim;
        }
    }
    auto result = Dataset::Make()->NumElements(nq)->Dim(dim)->Ids(ids)->Distances(dists)->Owner(true);
    result->Statistics(stats);
    return result;
}

// RangeSearch on top of the k-nearest search (range mode of BruteForce::SearchWithRequest,
// src/algorithm/bruteforce/bruteforce.cpp:388-545, and of FlatBucketSearcher,
// src/algorithm/ivf/flat_bucket_searcher.cpp:105-137): both keep a heap of limited_size entries (all
// vectors when it is negative) and push what lies within the radius, so the answer is the nearest
// limited_size of the in-radius vectors, ascending.  That is the k-nearest answer cut at the radius.
// Without a limit k grows until the answer is complete; past RANGE_K_MAX in-radius vectors (the scan's
// per-query candidate buffers bound k) the answer is fetched in pages: the vectors found so far are added
// to the search's inner-id deny bitmap and the next RANGE_K_MAX nearest are asked for, until a page reaches
// past the radius.  Pages are disjoint and each holds the nearest of what is left, so their concatenation
// is the ascending in-radius list.  `slack` is what the reference adds to the radius (THRESHOLD_ERROR for
// IVF, src/impl/searcher/basic_searcher.h:39; nothing for BruteForce).
constexpr int64_t RANGE_K_MAX = 512;

template <typename Knn>
DatasetPtr
range_over_knn(Knn&& knn, const DatasetPtr& query, int64_t n_live, float radius, float slack, int64_t limited_size,
               const vb200_filter* filter, const std::vector<int64_t>& label_of_inner) {
    check_argument(query != nullptr, "query is null");
    check_argument(query->GetNumElements() == 1, "query dataset should contain 1 vector only");
    check_argument(std::isfinite(radius), "radius must be finite");
    check_argument(radius >= 0.0f, "radius must be non-negative");
    check_argument(limited_size != 0, "limited_size must be greater than 0 or less than 0");
    if (n_live == 0) {
        return make_empty_result();
    }
    auto inside_of = [&](const DatasetPtr& found) {
        int64_t inside = 0;
        while (inside < found->GetDim() && found->GetDistances()[inside] <= radius + slack) {
            ++inside;
        }
        return inside;
    };
    auto pack = [&](const int64_t* src_ids, const float* src_dists, int64_t count, const std::string& stats) {
        auto* ids = new int64_t[static_cast<size_t>(std::max<int64_t>(count, 1))];
        auto* dists = new float[static_cast<size_t>(std::max<int64_t>(count, 1))];
        std::copy(src_ids, src_ids + count, ids);
        std::copy(src_dists, src_dists + count, dists);
        auto result = Dataset::Make()->NumElements(1)->Dim(count)->Ids(ids)->Distances(dists)->Owner(true);
        result->Statistics(stats);
        return result;
    };
    int64_t k = limited_size > 0 ? std::min(limited_size, n_live) : std::min<int64_t>(64, n_live);
    for (;;) {
        Expected<DatasetPtr> r = knn(k, filter);
        if (!r.has_value()) {
            fail(r.error().type, r.error().message);
        }
        const DatasetPtr& found = r.value();
        const int64_t got = found->GetDim();
        const int64_t inside = inside_of(found);
        const bool complete = limited_size > 0 || inside < got || got < k || k >= n_live;
        if (!complete && k < RANGE_K_MAX) {
            k = std::min({k * 8, RANGE_K_MAX, n_live});
            continue;
        }
        if (complete) {
            return pack(found->GetIds(), found->GetDistances(), inside, found->GetStatistics());
        }
        // every one of the RANGE_K_MAX nearest lies within the radius: go on in pages
        std::vector<int64_t> all_ids(found->GetIds(), found->GetIds() + inside);
        std::vector<float> all_dists(found->GetDistances(), found->GetDistances() + inside);
        std::unordered_map<int64_t, uint32_t> inner_of_label;
        inner_of_label.reserve(label_of_inner.size());
        for (size_t i = 0; i < label_of_inner.size(); ++i) {
            inner_of_label.emplace(label_of_inner[i], static_cast<uint32_t>(i));
        }
        std::vector<uint32_t> deny((label_of_inner.size() + 31) / 32, 0);
        if (filter != nullptr && filter->deny_inner_bits != nullptr) {
            const size_t words = std::min<size_t>(deny.size(), (filter->n_inner_bits + 31) / 32);
            std::copy(filter->deny_inner_bits, filter->deny_inner_bits + words, deny.begin());
        }
        vb200_filter paged = filter != nullptr ? *filter : vb200_filter{};
        paged.deny_inner_bits = deny.data();
        paged.n_inner_bits = label_of_inner.size();
        size_t marked = 0;
        std::string stats = found->GetStatistics();
        for (;;) {
            for (; marked < all_ids.size(); ++marked) {
                auto it = inner_of_label.find(all_ids[marked]);
                if (it != inner_of_label.end()) {
                    deny[it->second >> 5] |= 1u << (it->second & 31);
                }
            }
            Expected<DatasetPtr> page = knn(RANGE_K_MAX, &paged);
            if (!page.has_value()) {
                fail(page.error().type, page.error().message);
            }
            const DatasetPtr& next = page.value();
            const int64_t page_inside = inside_of(next);
            all_ids.insert(all_ids.end(), next->GetIds(), next->GetIds() + page_inside);
            all_dists.insert(all_dists.end(), next->GetDistances(), next->GetDistances() + page_inside);
            if (page_inside < next->GetDim() || next->GetDim() < RANGE_K_MAX) {
                break;
            }
        }
        return pack(all_ids.data(), all_dists.data(), static_cast<int64_t>(all_ids.size()), stats);
    }
}

// k beyond what one search of the engine returns (its per-query candidate buffers live in shared memory): the
// answer is fetched in pages like an unlimited range search -- what was found joins the deny bitmap, the next
// KNN_PAGE nearest are asked for -- one query at a time, since the bitmap belongs to a query.  `knn(one, k, f, i)`
// searches query i alone.
constexpr int64_t KNN_PAGE = 512;

template <typename Knn>
DatasetPtr
knn_in_pages(Knn&& knn, const DatasetPtr& query, int64_t dim, int64_t k, const vb200_filter* filter,
             const std::vector<int64_t>& label_of_inner) {
    check_argument(query != nullptr, "query is null");
    const int64_t nq = query->GetNumElements();
    check_argument(query->GetFloat32Vectors() != nullptr, "query vectors are null");
    std::unordered_map<int64_t, uint32_t> inner_of_label;
    inner_of_label.reserve(label_of_inner.size());
    for (size_t i = 0; i < label_of_inner.size(); ++i) {
        inner_of_label.emplace(label_of_inner[i], static_cast<uint32_t>(i));
    }
    auto* ids = new int64_t[static_cast<size_t>(std::max<int64_t>(nq * k, 1))];
    auto* dists = new float[static_cast<size_t>(std::max<int64_t>(nq * k, 1))];
    std::fill(ids, ids + nq * k, int64_t{-1});
    std::fill(dists, dists + nq * k, std::numeric_limits<float>::infinity());
    std::string stats;
    try {
        for (int64_t qi = 0; qi < nq; ++qi) {
            auto one = Dataset::Make()->NumElements(1)->Dim(dim)->Float32Vectors(query->GetFloat32Vectors() + qi * dim)->Owner(false);
            std::vector<uint32_t> deny((label_of_inner.size() + 31) / 32, 0);
            if (filter != nullptr && filter->deny_inner_bits != nullptr) {
                const size_t words = std::min<size_t>(deny.size(), (filter->n_inner_bits + 31) / 32);
                std::copy(filter->deny_inner_bits, filter->deny_inner_bits + words, deny.begin());
            }
            vb200_filter paged = filter != nullptr ? *filter : vb200_filter{};
            paged.deny_inner_bits = deny.data();
            paged.n_inner_bits = label_of_inner.size();
            int64_t have = 0;
            while (have < k) {
                const int64_t want = std::min<int64_t>(KNN_PAGE, k - have);
                Expected<DatasetPtr> page = knn(one, want, &paged, qi);
                if (!page.has_value()) {
                    fail(page.error().type, page.error().message);
                }
                const DatasetPtr& found = page.value();
                stats = found->GetStatistics();
                const int64_t got = found->GetDim();
                for (int64_t j = 0; j < got; ++j) {
                    ids[qi * k + have + j] = found->GetIds()[j];
                    dists[qi * k + have + j] = found->GetDistances()[j];
                    auto it = inner_of_label.find(found->GetIds()[j]);
                    if (it != inner_of_label.end()) {
                        deny[it->second >> 5] |= 1u << (it->second & 31);
                    }
                }
                have += got;
                if (got < want) {
                    break;
                }
            }
        }
    } catch (...) {
        delete[] ids;
        delete[] dists;
        throw;
    }
    return pack_result(ids, dists, nq, k, stats);
}

// A random orthogonal matrix with determinant +1, standing in for
// RandomOrthogonalMatrix::GenerateRandomOrthogonalMatrix (src/impl/transform/
// random_orthogonal_transformer.cpp:98-149): Gaussian entries from a seeded mt19937, then
// Gram-Schmidt (twice, in double) instead of LAPACK QR.
std::vector<float>
random_rotation(uint32_t dim, uint32_t seed) {
    std::mt19937 gen(seed);
    std::normal_distribution<float> dist(0.0f, 1.0f);
    std::vector<double> m(static_cast<size_t>(dim) * dim);
    for (auto& v : m) {
        v = dist(gen);
    }
    for (uint32_t i = 0; i < dim; ++i) {
        double* row = m.data() + static_cast<size_t>(i) * dim;
        for (int pass = 0; pass < 2; ++pass) {
            for (uint32_t j = 0; j < i; ++j) {
                const double* prev = m.data() + static_cast<size_t>(j) * dim;
                double dot = 0.0;
                for (uint32_t d = 0; d < dim; ++d) {
                    dot += row[d] * prev[d];
                }
                for (uint32_t d = 0; d < dim; ++d) {
                    row[d] -= dot * prev[d];
                }
            }
        }
        double norm = 0.0;
        for (uint32_t d = 0; d < dim; ++d) {
            norm += row[d] * row[d];
        }
        norm = std::sqrt(norm);
        if (norm < 1e-12) {
            fail(ErrorType::INTERNAL_ERROR, "degenerate random matrix");
        }
        for (uint32_t d = 0; d < dim; ++d) {
            row[d] /= norm;
        }
    }
    std::vector<float> out(m.size());
    for (size_t i = 0; i < m.size(); ++i) {
        out[i] = static_cast<float>(m[i]);
    }
    return out;
}

}  // namespace

// -------------------------------------------------------------------------------------------------
// Dataset
// -------------------------------------------------------------------------------------------------
DatasetPtr
Dataset::Make() {
    return DatasetPtr(new Dataset());
}

Dataset::~Dataset() {
    if (owner_) {
        delete[] ids_;
        delete[] distances_;
        delete[] vectors_;
        delete[] half_vectors_;
    }
}

DatasetPtr Dataset::Owner(bool is_owner) { owner_ = is_owner; return shared_from_this(); }
DatasetPtr Dataset::NumElements(int64_t n) { num_elements_ = n; return shared_from_this(); }
DatasetPtr Dataset::Dim(int64_t dim) { dim_ = dim; return shared_from_this(); }
DatasetPtr Dataset::Ids(const int64_t* ids) { ids_ = ids; return shared_from_this(); }
DatasetPtr Dataset::Distances(const float* dists) { distances_ = dists; return shared_from_this(); }
DatasetPtr Dataset::Float32Vectors(const float* v) { vectors_ = v; return shared_from_this(); }
DatasetPtr Dataset::Float16Vectors(const uint16_t* v) { half_vectors_ = v; return shared_from_this(); }
DatasetPtr Dataset::Statistics(const std::string& s) { statistics_ = s; return shared_from_this(); }

// -------------------------------------------------------------------------------------------------
// IVF
// -------------------------------------------------------------------------------------------------
namespace {

void
check_base(const DatasetPtr& base, uint32_t dim, bool need_ids) {
    check_argument(base != nullptr, "dataset is null");
    check_argument(base->GetNumElements() >= 0, "dataset has a negative element count");
    if (base->GetNumElements() == 0) {
        return;
    }
    if (base->GetDim() != static_cast<int64_t>(dim)) {
        fail(ErrorType::DIMENSION_NOT_EQUAL,
             "dimension of the dataset (" + std::to_string(base->GetDim()) + ") is not equal to the index (" +
                 std::to_string(dim) + ")");
    }
    check_argument(base->GetFloat32Vectors() != nullptr, "dataset has no float32 vectors");
    check_argument(!need_ids || base->GetIds() != nullptr, "dataset has no ids");
}

class GpuIVF : public Index {
public:
    GpuIVF(const CommonParam& common) : dim_(common.dim), metric_(common.metric) {
        const Json& p = common.index_param;
        // External keys of IVF::CheckAndMappingExternalParam (src/algorithm/ivf/ivf.cpp:140-395)
        // with the defaults of its template (:78-135).
        static const std::set<std::string> known = {
            "buckets_count", "base_quantization_type", "base_io_type", "base_file_path", "precise_io_type",
            "precise_file_path", "precise_quantization_type", "ivf_train_type", "partition_strategy_type",
            "use_reorder", "buckets_per_data", "thread_count", "train_sample_count", "use_residual",
            "rabitq_bits_per_dim_query", "rabitq_bits_per_dim_base", "rabitq_version", "rabitq_use_fht",
            "rabitq_pca_dim", "use_attribute_filter", "first_order_buckets_count",
            "second_order_buckets_count"};
        check_known_keys(p, known, "index_param of ivf");
        int64_t buckets = get_int(p, "buckets_count", 10);
        check_argument(buckets >= 1, "buckets_count must be at least 1");
        nlist_ = static_cast<uint32_t>(buckets);
        std::string quant = get_string(p, "base_quantization_type", "fp32");
        if (quant == "sq8") {
            quant_ = VB200_QUANT_SQ8;
        } else if (quant == "rabitq") {
            quant_ = VB200_QUANT_RABITQ;
        } else if (quant == "fp32") {
            quant_ = VB200_QUANT_FP32;
        } else if (quant == "bf16") {
            quant_ = VB200_QUANT_BF16;
        } else if (quant == "fp16") {
            quant_ = VB200_QUANT_FP16;
        } else if (quant == "sq8_uniform") {
            quant_ = VB200_QUANT_SQ8_UNIFORM;
        } else {
            fail(ErrorType::INVALID_ARGUMENT,
                 "base_quantization_type \"" + quant +
                     "\" is not served by the GPU engine (fp32, bf16, fp16, sq8, sq8_uniform and rabitq are)");
        }
        use_reorder_ = get_bool(p, "use_reorder", false);
        std::string precise = get_string(p, "precise_quantization_type", "fp32");
        check_argument(precise == "fp32", "precise_quantization_type must be fp32 for the GPU engine");
        std::string train_type = get_string(p, "ivf_train_type", "kmeans");
        check_argument(train_type == "kmeans" || train_type == "random",
                       "ivf_train_type must be kmeans or random, got " + train_type);
        kmeans_iters_ = train_type == "kmeans" ? 25 : 0;  // IVFNearestPartition::Train hard-codes 25
        check_argument(get_string(p, "partition_strategy_type", "ivf") == "ivf",
                       "partition_strategy_type must be ivf for the GPU engine (gno_imi is out of scope)");
        buckets_per_data_ = get_int(p, "buckets_per_data", 1);
        check_argument(buckets_per_data_ >= 1 && buckets_per_data_ <= std::min<int64_t>(nlist_, 16),
                       "buckets_per_data must lie in [1, min(buckets_count, 16)]");
        check_argument(get_int(p, "thread_count", 1) >= 1, "thread_count must be positive");
        use_residual_ = get_bool(p, "use_residual", false);
        check_argument(!use_residual_ || quant_ == VB200_QUANT_SQ8,
                       "use_residual is served by the GPU engine for sq8 buckets only");
        check_argument(!get_bool(p, "use_attribute_filter", false),
                       "use_attribute_filter is not served by the GPU engine");
        check_argument(get_int(p, "rabitq_bits_per_dim_query", 32) == 32 &&
                           get_int(p, "rabitq_bits_per_dim_base", 1) == 1,
                       "the GPU engine serves rabitq with a 32-bit query and 1-bit base codes");
        check_argument(get_string(p, "rabitq_version", "standard") == "standard" &&
                           !get_bool(p, "rabitq_use_fht", false) && get_int(p, "rabitq_pca_dim", 0) == 0,
                       "the GPU engine serves the standard rabitq layout without FHT or PCA");
        // default of IVFParameter (src/algorithm/ivf/ivf_parameter.cpp:88-98)
        int64_t def_sample = std::max<int64_t>(65536, 64 * static_cast<int64_t>(nlist_));
        train_sample_count_ = get_int(p, "train_sample_count", def_sample);
        check_argument(train_sample_count_ >= 512, "train_sample_count must be at least 512");
        check_status(vb200_ivf_create(dim_, metric_, nlist_, quant_, use_reorder_ ? 1 : 0, &handle_));
        if (buckets_per_data_ > 1) {
            check_status(vb200_ivf_set_buckets_per_data(handle_, static_cast<uint32_t>(buckets_per_data_)));
        }
        if (use_residual_) {
            check_status(vb200_ivf_set_use_residual(handle_, 1));
        }
        if (quant_ == VB200_QUANT_RABITQ) {
            rotation_ = random_rotation(dim_, 47);
            check_status(vb200_ivf_set_rabitq_rotation(handle_, rotation_.data()));
        }
    }

    ~GpuIVF() override {
        vb200_ivf_destroy(handle_);
    }

    Expected<std::vector<int64_t>>
    Build(const DatasetPtr& base) override {
        return safe_call<std::vector<int64_t>>([&]() {
            std::lock_guard<std::mutex> lock(mu_);
            check_base(base, dim_, true);
            if (vb200_ivf_num_elements(handle_) > 0 || built_) {
                fail(ErrorType::BUILD_TWICE, "index has been build, cannot build again");
            }
            if (base->GetNumElements() == 0) {
                return std::vector<int64_t>{};
            }
            train_locked(base);
            add_locked(base);
            built_ = true;
            return std::vector<int64_t>{};
        });
    }

    Expected<void*>
    Train(const DatasetPtr& data) override {
        return safe_call<void*>([&]() -> void* {
            std::lock_guard<std::mutex> lock(mu_);
            check_base(data, dim_, false);
            check_argument(data->GetNumElements() > 0, "training data is empty");
            train_locked(data);
            return nullptr;
        });
    }

    Expected<std::vector<int64_t>>
    Add(const DatasetPtr& base) override {
        return safe_call<std::vector<int64_t>>([&]() {
            std::lock_guard<std::mutex> lock(mu_);
            check_base(base, dim_, true);
            if (base->GetNumElements() == 0) {
                return std::vector<int64_t>{};
            }
            if (!trained_) {  // the reference trains on the first batch too (IVF::Add -> Train)
                train_locked(base);
            }
            add_locked(base);
            return std::vector<int64_t>{};
        });
    }

    Expected<DatasetPtr>
    KnnSearch(const DatasetPtr& query, int64_t k, const std::string& parameters) const override {
        return knn_impl(query, k, parameters, nullptr);
    }

    Expected<DatasetPtr>
    KnnSearch(const DatasetPtr& query, int64_t k, const std::string& parameters, BitsetPtr invalid) const override {
        if (invalid == nullptr || invalid->Words().empty()) {
            return knn_impl(query, k, parameters, nullptr);
        }
        vb200_filter f{invalid->Words().data(), invalid->Words().size() * 64, nullptr, 0};
        return knn_impl(query, k, parameters, &f);
    }

    Expected<DatasetPtr>
    KnnSearch(const DatasetPtr& query, int64_t k, const std::string& parameters,
              const std::function<bool(int64_t)>& filter) const override {
        if (!filter) {
            return knn_impl(query, k, parameters, nullptr);
        }
        // the callback is evaluated once per stored vector and becomes a bitmap over insertion order
        std::vector<uint32_t> deny((labels_host_.size() + 31) / 32, 0);
        for (size_t i = 0; i < labels_host_.size(); ++i) {
            if (filter(labels_host_[i])) {
                deny[i >> 5] |= 1u << (i & 31);
            }
        }
        vb200_filter f{nullptr, 0, deny.data(), labels_host_.size()};
        return knn_impl(query, k, parameters, &f);
    }

    Expected<uint32_t>
    Remove(const std::vector<int64_t>& ids) override {
        return safe_call<uint32_t>([&]() {
            std::lock_guard<std::mutex> lock(mu_);
            uint64_t removed = 0;
            check_status(remove_labels(ids.data(), ids.size(), &removed));
            removed_labels_.insert(removed_labels_.end(), ids.begin(), ids.end());
            return static_cast<uint32_t>(removed);
        });
    }

    Expected<DatasetPtr>
    RangeSearch(const DatasetPtr& query, float radius, const std::string& parameters,
                int64_t limited_size) const override {
        return range_impl(query, radius, parameters, limited_size, nullptr);
    }

    Expected<DatasetPtr>
    RangeSearch(const DatasetPtr& query, float radius, const std::string& parameters, BitsetPtr invalid,
                int64_t limited_size) const override {
        if (invalid == nullptr || invalid->Words().empty()) {
            return range_impl(query, radius, parameters, limited_size, nullptr);
        }
        vb200_filter f{invalid->Words().data(), invalid->Words().size() * 64, nullptr, 0};
        return range_impl(query, radius, parameters, limited_size, &f);
    }

    Expected<DatasetPtr>
    RangeSearch(const DatasetPtr& query, float radius, const std::string& parameters,
                const std::function<bool(int64_t)>& filter, int64_t limited_size) const override {
        if (!filter) {
            return range_impl(query, radius, parameters, limited_size, nullptr);
        }
        std::vector<uint32_t> deny((labels_host_.size() + 31) / 32, 0);
        for (size_t i = 0; i < labels_host_.size(); ++i) {
            if (filter(labels_host_[i])) {
                deny[i >> 5] |= 1u << (i & 31);
            }
        }
        vb200_filter f{nullptr, 0, deny.data(), labels_host_.size()};
        return range_impl(query, radius, parameters, limited_size, &f);
    }

    // IVF::SearchWithRequest (src/algorithm/ivf/ivf.cpp:2052-2354): the request's filters become the
    // engine's id filter (a bitset marks ids that are filtered out, filter_ says which ids are valid),
    // bucket_ids_ replaces routing after the reference's checks, range mode takes one query.
    Expected<DatasetPtr>
    SearchWithRequest(const SearchRequest& request) const override {
        std::vector<uint32_t> deny;
        vb200_filter f{nullptr, 0, nullptr, 0};
        bool filtered = false;
        if (request.enable_bitset_filter_ && request.bitset_filter_ != nullptr && !request.bitset_filter_->Words().empty()) {
            f.invalid_label_bits = request.bitset_filter_->Words().data();
            f.n_label_bits = request.bitset_filter_->Words().size() * 64;
            filtered = true;
        }
        if (request.enable_filter_ && request.filter_) {
            deny.assign((labels_host_.size() + 31) / 32, 0);
            for (size_t i = 0; i < labels_host_.size(); ++i) {
                if (!request.filter_(labels_host_[i])) {
                    deny[i >> 5] |= 1u << (i & 31);
                }
            }
            f.deny_inner_bits = deny.data();
            f.n_inner_bits = labels_host_.size();
            filtered = true;
        }
        const vb200_filter* fp = filtered ? &f : nullptr;
        const auto* buckets = request.bucket_ids_.empty() ? nullptr : &request.bucket_ids_;
        if (request.mode_ == SearchMode::RANGE_SEARCH) {
            return range_impl(request.query_, request.radius_, request.params_str_, request.limited_size_, fp, buckets);
        }
        return knn_impl(request.query_, request.topk_, request.params_str_, fp, buckets);
    }

    Expected<DatasetPtr>
    range_impl(const DatasetPtr& query, float radius, const std::string& parameters, int64_t limited_size,
               const vb200_filter* filter, const std::vector<std::vector<int64_t>>* bucket_ids = nullptr) const {
        return safe_call<DatasetPtr>([&]() {
            return range_over_knn(
                [&](int64_t k, const vb200_filter* f) { return knn_impl(query, k, parameters, f, bucket_ids); }, query,
                GetNumElements(), radius, 2e-6f, limited_size, filter, labels_host_);
        });
    }

    Expected<void>
    Serialize(std::ostream& out) const override {
        return safe_void([&]() {
            std::lock_guard<std::mutex> lock(mu_);
            write_header(out, file_header());
            write_pod<uint32_t>(out, trained_ ? 1 : 0);
            const uint64_t n_total = labels_host_.size();
            write_pod<uint64_t>(out, n_total);
            if (trained_) {
                std::vector<float> centroids(static_cast<size_t>(nlist_) * dim_);
                check_status(vb200_ivf_get_centroids(handle_, centroids.data()));
                write_array(out, centroids);
                if (quant_ == VB200_QUANT_SQ8) {
                    std::vector<float> lower(dim_), diff(dim_);
                    check_status(vb200_ivf_get_sq8_model(handle_, lower.data(), diff.data()));
                    write_array(out, lower);
                    write_array(out, diff);
                } else if (quant_ == VB200_QUANT_SQ8_UNIFORM) {
                    std::vector<float> model(2);
                    check_status(vb200_ivf_get_sq8_uniform_model(handle_, &model[0], &model[1]));
                    write_array(out, model);
                } else if (quant_ == VB200_QUANT_RABITQ) {
                    std::vector<float> centre(dim_);
                    check_status(vb200_ivf_get_rabitq_centroid(handle_, centre.data()));
                    write_array(out, rotation_);
                    write_array(out, centre);
                }
            }
            if (n_total > 0) {
                std::vector<int64_t> sizes(nlist_);
                check_status(vb200_ivf_get_lists(handle_, sizes.data(), nullptr, nullptr));
                uint64_t total = 0;
                for (int64_t v : sizes) {
                    total += static_cast<uint64_t>(v);
                }
                std::vector<uint8_t> codes(total * static_cast<uint64_t>(code_size()));
                std::vector<int64_t> inner(total);
                check_status(vb200_ivf_get_lists(handle_, nullptr, codes.data(), inner.data()));
                write_array(out, sizes);
                write_array(out, codes);
                write_array(out, inner);
                write_array(out, labels_host_);
                if (use_reorder_) {
                    std::vector<float> rows(n_total * dim_);
                    check_status(vb200_ivf_get_rows(handle_, rows.data()));
                    write_array(out, rows);
                }
            }
            write_array(out, removed_labels_);
            check_stream_written(out);
        });
    }

    Expected<void>
    Deserialize(std::istream& in) override {
        return safe_void([&]() {
            std::lock_guard<std::mutex> lock(mu_);
            if (trained_ || !labels_host_.empty()) {
                fail(ErrorType::INDEX_NOT_EMPTY, "failed to Deserialize: index is not empty");
            }
            read_header(in, file_header());
            const bool trained = read_pod<uint32_t>(in) != 0;
            const uint64_t n_total = read_pod<uint64_t>(in);
            if (!trained && n_total > 0) {
                fail(ErrorType::INVALID_BINARY, "index stream: vectors without a trained model");
            }
            if (trained) {
                auto centroids = read_array<float>(in, static_cast<uint64_t>(nlist_) * dim_, "centroids");
                check_status(vb200_ivf_set_centroids(handle_, centroids.data()));
                if (quant_ == VB200_QUANT_SQ8) {
                    auto lower = read_array<float>(in, dim_, "sq8 lower bound");
                    auto diff = read_array<float>(in, dim_, "sq8 diff");
                    check_status(vb200_ivf_set_sq8_model(handle_, lower.data(), diff.data()));
                } else if (quant_ == VB200_QUANT_SQ8_UNIFORM) {
                    auto model = read_array<float>(in, 2, "sq8_uniform model");
                    check_status(vb200_ivf_set_sq8_uniform_model(handle_, model[0], model[1]));
                } else if (quant_ == VB200_QUANT_RABITQ) {
                    auto rotation = read_array<float>(in, static_cast<uint64_t>(dim_) * dim_, "rabitq rotation");
                    auto centre = read_array<float>(in, dim_, "rabitq centroid");
                    check_status(vb200_ivf_set_rabitq_rotation(handle_, rotation.data()));
                    check_status(vb200_ivf_set_rabitq_centroid(handle_, centre.data()));
                    rotation_ = std::move(rotation);
                }
                trained_ = true;
            }
            if (n_total > 0) {
                auto sizes = read_array<int64_t>(in, nlist_, "list sizes");
                uint64_t total = 0;
                for (int64_t v : sizes) {
                    if (v < 0) {
                        fail(ErrorType::INVALID_BINARY, "index stream: negative list size");
                    }
                    total += static_cast<uint64_t>(v);
                }
                auto codes = read_array<uint8_t>(in, total * static_cast<uint64_t>(code_size()), "codes");
                auto inner = read_array<int64_t>(in, total, "inner ids");
                auto labels = read_array<int64_t>(in, n_total, "labels");
                std::vector<float> rows;
                if (use_reorder_) {
                    rows = read_array<float>(in, n_total * dim_, "reorder rows");
                }
                check_status(vb200_ivf_set_lists(handle_, sizes.data(), codes.data(), inner.data(), labels.data(),
                                                 n_total, use_reorder_ ? rows.data() : nullptr));
                labels_host_ = std::move(labels);
                built_ = true;
            }
            auto removed = read_array_any<int64_t>(in, "removed labels");
            check_end_mark(in);
            if (!removed.empty()) {
                check_status(remove_labels(removed.data(), removed.size(), nullptr));
                removed_labels_ = std::move(removed);
            }
        });
    }

    Expected<DatasetPtr>
    knn_impl(const DatasetPtr& query, int64_t k, const std::string& parameters, const vb200_filter* filter,
             const std::vector<std::vector<int64_t>>* bucket_ids = nullptr) const {
        if (k <= KNN_PAGE || query == nullptr || query->GetNumElements() == 0 || vb200_ivf_num_elements(handle_) == 0) {
            return knn_page(query, k, parameters, filter, bucket_ids);
        }
        return safe_call<DatasetPtr>([&]() {
            check_base(query, dim_, false);
            const bool listed = bucket_ids != nullptr && !bucket_ids->empty();
            check_argument(!listed || static_cast<int64_t>(bucket_ids->size()) == query->GetNumElements(),
                           "bucket_ids_ size must match the number of query vectors");
            return knn_in_pages(
                [&](const DatasetPtr& one, int64_t kk, const vb200_filter* f, int64_t qi) {
                    if (!listed) {
                        return knn_page(one, kk, parameters, f, nullptr);
                    }
                    std::vector<std::vector<int64_t>> mine{(*bucket_ids)[static_cast<size_t>(qi)]};
                    return knn_page(one, kk, parameters, f, &mine);
                },
                query, dim_, k, filter, labels_host_);
        });
    }

    Expected<DatasetPtr>
    knn_page(const DatasetPtr& query, int64_t k, const std::string& parameters, const vb200_filter* filter,
             const std::vector<std::vector<int64_t>>* bucket_ids = nullptr) const {
        return safe_call<DatasetPtr>([&]() {
            check_argument(query != nullptr, "query is null");
            check_argument(k > 0, "k must be greater than 0");
            // IVFSearchParameters::FromJson (src/algorithm/ivf/ivf_parameter.cpp:150-187)
            Json root = Json::Parse(parameters);
            check_argument(root.IsObject() && root.Contains("ivf"), "parameters must contains ivf");
            const Json& ivf = root.At("ivf");
            check_argument(ivf.IsObject() && ivf.Contains("scan_buckets_count"),
                           "parameters[ivf] must contains scan_buckets_count");
            int64_t nprobe = get_int(ivf, "scan_buckets_count", 1);
            check_argument(nprobe >= 1, "scan_buckets_count must be positive");
            double factor = get_number(ivf, "factor", 2.0);
            bool disable_scan = get_bool(ivf, "disable_bucket_scan", false);
            // IndexSearchParameter::FromJson (src/algorithm/index_search_parameter.h:27-48): enable_reorder
            // (default true), timeout_ms (an integer; present = the search is timed), parallelism (host threads
            // of the reference's scan: nothing to do here).  Keys it does not know are ignored, as there.
            vb200_search_options options{};
            options.enable_reorder = get_bool(ivf, "enable_reorder", true) ? 1 : 0;
            options.has_timeout = ivf.Contains("timeout_ms") ? 1 : 0;
            options.timeout_ms = options.has_timeout != 0 ? static_cast<double>(get_int(ivf, "timeout_ms", 0)) : 0.0;
            if (query->GetNumElements() == 0 || vb200_ivf_num_elements(handle_) == 0) {
                return make_empty_result();
            }
            check_base(query, dim_, false);
            const int64_t nq = query->GetNumElements();
            // SearchRequest::bucket_ids_: the checks of IVF::SearchWithRequest (src/algorithm/ivf/ivf.cpp:2075-2112),
            // then one row of bucket ids per query, padded with -1 to the longest list
            std::vector<int32_t> buckets_flat;
            if (bucket_ids != nullptr && !bucket_ids->empty()) {
                check_argument(static_cast<int64_t>(bucket_ids->size()) == nq,
                               "bucket_ids_ size must match the number of query vectors; got " +
                                   std::to_string(bucket_ids->size()) + " bucket lists for " + std::to_string(nq) +
                                   " queries");
                check_argument(!disable_scan, "bucket_ids_ is incompatible with disable_bucket_scan mode");
                size_t longest = 0;
                for (size_t qi = 0; qi < bucket_ids->size(); ++qi) {
                    const auto& ids = (*bucket_ids)[qi];
                    check_argument(!ids.empty(), "bucket_ids_[" + std::to_string(qi) +
                                                     "] must not be empty; use empty outer vector for default routing");
                    std::vector<int64_t> seen(ids);
                    std::sort(seen.begin(), seen.end());
                    for (size_t i = 0; i < seen.size(); ++i) {
                        check_argument(seen[i] >= 0 && seen[i] < static_cast<int64_t>(nlist_),
                                       "bucket_id " + std::to_string(seen[i]) + " out of range [0, " +
                                           std::to_string(nlist_) + ")");
                        check_argument(i == 0 || seen[i] != seen[i - 1], "duplicate bucket_id " + std::to_string(seen[i]));
                    }
                    longest = std::max(longest, ids.size());
                }
                buckets_flat.assign(static_cast<size_t>(nq) * longest, -1);
                for (size_t qi = 0; qi < bucket_ids->size(); ++qi) {
                    for (size_t i = 0; i < (*bucket_ids)[qi].size(); ++i) {
                        buckets_flat[qi * longest + i] = static_cast<int32_t>((*bucket_ids)[qi][i]);
                    }
                }
                nprobe = static_cast<int64_t>(longest);
            }
            if (disable_scan) {
                // routing only: bucket ids with their centroid distances (IVF::route_buckets_only,
                // src/algorithm/ivf/ivf.cpp:1589-1660)
                int64_t np = std::min<int64_t>(nprobe, nlist_);
                std::vector<int32_t> buckets(static_cast<size_t>(nq * np));
                auto* dists = new float[static_cast<size_t>(nq * np)];
                auto* ids = new int64_t[static_cast<size_t>(nq * np)];
                int status = vb200_ivf_route(handle_, query->GetFloat32Vectors(), nq, static_cast<uint32_t>(np),
                                             buckets.data(), dists);
                if (status != 0) {
                    delete[] dists;
                    delete[] ids;
                    check_status(status);
                }
                for (size_t i = 0; i < buckets.size(); ++i) {
                    ids[i] = buckets[i];
                }
                return Dataset::Make()->NumElements(nq)->Dim(np)->Ids(ids)->Distances(dists)->Owner(true);
            }
            auto* ids = new int64_t[static_cast<size_t>(nq * k)];
            auto* dists = new float[static_cast<size_t>(nq * k)];
            int timed_out = 0;
            int status = vb200_ivf_search_ex(handle_, query->GetFloat32Vectors(), nq, static_cast<uint32_t>(k),
                                             static_cast<uint32_t>(std::min<int64_t>(nprobe, 0x7fffffff)),
                                             static_cast<float>(factor),
                                             buckets_flat.empty() ? nullptr : buckets_flat.data(), filter, &options, ids,
                                             dists, &timed_out);
            if (status != 0) {
                delete[] ids;
                delete[] dists;
                check_status(status);
            }
            int64_t scanned = vb200_ivf_last_scan_bytes(handle_);
            // the fields of QueryStats a caller reads back (dist_cmp, is_timeout)
            std::string stats = "{\"dist_cmp\":" + std::to_string(code_size() > 0 ? scanned / code_size() : 0) +
                                ",\"is_timeout\":" + (timed_out != 0 ? "true" : "false") + "}";
            return pack_result(ids, dists, nq, k, stats);
        });
    }

    int64_t GetNumElements() const override { return vb200_ivf_num_elements(handle_); }
    int64_t GetMemoryUsage() const override { return vb200_ivf_memory_usage(handle_); }
    std::string GetIndexType() const override { return "ivf"; }

private:
    int64_t
    code_size() const {
        if (quant_ == VB200_QUANT_FP32) {
            return static_cast<int64_t>(dim_) * 4;
        }
        if (quant_ == VB200_QUANT_BF16 || quant_ == VB200_QUANT_FP16) {
            return static_cast<int64_t>(dim_) * 2;
        }
        if (quant_ == VB200_QUANT_SQ8_UNIFORM) {
            const int64_t align = metric_ == VB200_METRIC_L2 ? 8 : 4;   // sq8_uniform_quantizer.cpp:32-60
            return (static_cast<int64_t>(dim_) + align - 1) / align * align + align;
        }
        return quant_ == VB200_QUANT_SQ8 ? dim_ : static_cast<int64_t>(vb200_rabitq_code_size(dim_));
    }

    void
    train_locked(const DatasetPtr& data) {
        if (trained_) {
            return;
        }
        const int64_t n = data->GetNumElements();
        const float* x = data->GetFloat32Vectors();
        if (n < static_cast<int64_t>(nlist_)) {
            fail(ErrorType::INVALID_ARGUMENT, "k cannot be larger than count");
        }
        // sample_train_data (src/utils/util_functions.cpp:273-330) draws a reservoir sample from
        // std::random_device; here a strided sample of the same size (all rows when they fit).
        std::vector<float> sample;
        int64_t count = n;
        if (n > train_sample_count_) {
            count = std::max<int64_t>(train_sample_count_, nlist_);
            sample.resize(static_cast<size_t>(count) * dim_);
            const int64_t stride = n / count;
            for (int64_t j = 0; j < count; ++j) {
                std::memcpy(sample.data() + static_cast<size_t>(j) * dim_, x + static_cast<size_t>(j * stride) * dim_,
                            dim_ * sizeof(float));
            }
            x = sample.data();
        }
        // KMeansCluster::Run seeds with k-means++ (src/impl/cluster/kmeans_cluster.h:47); the
        // generator's seed is fixed here so that a build is reproducible.
        std::vector<float> seeds;
        if (kmeans_iters_ > 0) {
            seeds.resize(static_cast<size_t>(nlist_) * dim_);
            check_status(vb200_kmeans_init(x, static_cast<uint64_t>(count), static_cast<uint32_t>(dim_), nlist_,
                                           KMEANS_SEED, seeds.data(), nullptr));
        }
        check_status(vb200_ivf_train(handle_, x, static_cast<uint64_t>(count), kmeans_iters_,
                                     seeds.empty() ? nullptr : seeds.data()));
        trained_ = true;
    }

    void
    add_locked(const DatasetPtr& base) {
        check_status(vb200_ivf_add(handle_, base->GetFloat32Vectors(), static_cast<uint64_t>(base->GetNumElements()),
                                   base->GetIds(), nullptr));
        labels_host_.insert(labels_host_.end(), base->GetIds(), base->GetIds() + base->GetNumElements());
    }

    int
    remove_labels(const int64_t* ids, uint64_t count, uint64_t* removed) {
        return vb200_ivf_remove(handle_, ids, count, removed);
    }

    FileHeader
    file_header() const {
        // the flag word also carries use_residual and buckets_per_data, so that a file is only loaded into an index created alike
        return FileHeader{FILE_KIND_IVF, dim_, nlist_, (use_reorder_ ? 1u : 0u) | (use_residual_ ? 2u : 0u) | (static_cast<uint32_t>(buckets_per_data_ - 1) << 8),
                          metric_, quant_};
    }

    std::vector<int64_t> labels_host_;     // ids in insertion order, for callback filters
    std::vector<int64_t> removed_labels_;  // every id Remove was asked for, replayed after a reload
    std::vector<float> rotation_;          // RaBitQ: the rotation in use

    uint32_t dim_;
    int metric_;
    int64_t buckets_per_data_ = 1;
    bool use_residual_ = false;
    static constexpr uint32_t KMEANS_SEED = 47;
    uint32_t nlist_ = 10;
    int quant_ = VB200_QUANT_SQ8;
    bool use_reorder_ = false;
    int kmeans_iters_ = 25;
    int64_t train_sample_count_ = 65536;
    bool trained_ = false;
    bool built_ = false;
    vb200_ivf_t handle_ = nullptr;
    mutable std::mutex mu_;
};

// -------------------------------------------------------------------------------------------------
// BruteForce
// -------------------------------------------------------------------------------------------------
class GpuBruteForce : public Index {
public:
    GpuBruteForce(const CommonParam& common) : dim_(common.dim), metric_(common.metric) {
        const Json& p = common.index_param;
        // External keys of BruteForce::CheckAndMappingExternalParam
        // (src/algorithm/bruteforce/bruteforce.cpp:1273-1361).
        static const std::set<std::string> known = {"base_quantization_type", "base_io_type", "base_file_path",
                                                    "thread_count", "resize_increase_count_bit",
                                                    "use_attribute_filter", "store_raw_vector"};
        check_known_keys(p, known, "index_param of brute_force");
        std::string quant = get_string(p, "base_quantization_type", "fp32");
        if (quant == "fp32") {
            quant_ = VB200_QUANT_FP32;
        } else if (quant == "bf16") {
            quant_ = VB200_QUANT_BF16;
        } else {
            fail(ErrorType::INVALID_ARGUMENT, "base_quantization_type \"" + quant +
                                                  "\" is not served by the GPU engine (fp32 and bf16 are)");
        }
        check_argument(!get_bool(p, "use_attribute_filter", false),
                       "use_attribute_filter is not served by the GPU engine");
        check_status(vb200_bf_create(dim_, metric_, quant_, &handle_));
    }

    ~GpuBruteForce() override {
        vb200_bf_destroy(handle_);
    }

    Expected<std::vector<int64_t>>
    Build(const DatasetPtr& base) override {
        return safe_call<std::vector<int64_t>>([&]() {
            std::lock_guard<std::mutex> lock(mu_);
            if (vb200_bf_num_elements(handle_) > 0) {
                fail(ErrorType::BUILD_TWICE, "index has been build, cannot build again");
            }
            add_locked(base);
            return std::vector<int64_t>{};
        });
    }

    Expected<void*>
    Train(const DatasetPtr&) override {
        return Expected<void*>(nullptr);  // fp32 / bf16 codecs have nothing to train (bruteforce.cpp:91-95)
    }

    Expected<std::vector<int64_t>>
    Add(const DatasetPtr& base) override {
        return safe_call<std::vector<int64_t>>([&]() {
            std::lock_guard<std::mutex> lock(mu_);
            add_locked(base);
            return std::vector<int64_t>{};
        });
    }

    Expected<DatasetPtr>
    KnnSearch(const DatasetPtr& query, int64_t k, const std::string& parameters) const override {
        return knn_impl(query, k, parameters, nullptr);
    }

    Expected<DatasetPtr>
    KnnSearch(const DatasetPtr& query, int64_t k, const std::string& parameters, BitsetPtr invalid) const override {
        if (invalid == nullptr || invalid->Words().empty()) {
            return knn_impl(query, k, parameters, nullptr);
        }
        vb200_filter f{invalid->Words().data(), invalid->Words().size() * 64, nullptr, 0};
        return knn_impl(query, k, parameters, &f);
    }

    Expected<DatasetPtr>
    KnnSearch(const DatasetPtr& query, int64_t k, const std::string& parameters,
              const std::function<bool(int64_t)>& filter) const override {
        if (!filter) {
            return knn_impl(query, k, parameters, nullptr);
        }
        // the callback is evaluated once per stored vector and becomes a bitmap over insertion order
        std::vector<uint32_t> deny((labels_host_.size() + 31) / 32, 0);
        for (size_t i = 0; i < labels_host_.size(); ++i) {
            if (filter(labels_host_[i])) {
                deny[i >> 5] |= 1u << (i & 31);
            }
        }
        vb200_filter f{nullptr, 0, deny.data(), labels_host_.size()};
        return knn_impl(query, k, parameters, &f);
    }

    Expected<uint32_t>
    Remove(const std::vector<int64_t>& ids) override {
        return safe_call<uint32_t>([&]() {
            std::lock_guard<std::mutex> lock(mu_);
            uint64_t removed = 0;
            check_status(remove_labels(ids.data(), ids.size(), &removed));
            removed_labels_.insert(removed_labels_.end(), ids.begin(), ids.end());
            return static_cast<uint32_t>(removed);
        });
    }

    Expected<DatasetPtr>
    RangeSearch(const DatasetPtr& query, float radius, const std::string& parameters,
                int64_t limited_size) const override {
        return range_impl(query, radius, parameters, limited_size, nullptr);
    }

    Expected<DatasetPtr>
    RangeSearch(const DatasetPtr& query, float radius, const std::string& parameters, BitsetPtr invalid,
                int64_t limited_size) const override {
        if (invalid == nullptr || invalid->Words().empty()) {
            return range_impl(query, radius, parameters, limited_size, nullptr);
        }
        vb200_filter f{invalid->Words().data(), invalid->Words().size() * 64, nullptr, 0};
        return range_impl(query, radius, parameters, limited_size, &f);
    }

    Expected<DatasetPtr>
    RangeSearch(const DatasetPtr& query, float radius, const std::string& parameters,
                const std::function<bool(int64_t)>& filter, int64_t limited_size) const override {
        if (!filter) {
            return range_impl(query, radius, parameters, limited_size, nullptr);
        }
        std::vector<uint32_t> deny((labels_host_.size() + 31) / 32, 0);
        for (size_t i = 0; i < labels_host_.size(); ++i) {
            if (filter(labels_host_[i])) {
                deny[i >> 5] |= 1u << (i & 31);
            }
        }
        vb200_filter f{nullptr, 0, deny.data(), labels_host_.size()};
        return range_impl(query, radius, parameters, limited_size, &f);
    }

    // BruteForce::SearchWithRequest (src/algorithm/bruteforce/bruteforce.cpp:370-635): KNN or range search
    // with the request's filters; bucket lists have no meaning here and are rejected.
    Expected<DatasetPtr>
    SearchWithRequest(const SearchRequest& request) const override {
        if (!request.bucket_ids_.empty()) {
            return Error{ErrorType::INVALID_ARGUMENT, "bucket_ids_ is only supported by the ivf index"};
        }
        std::vector<uint32_t> deny;
        vb200_filter f{nullptr, 0, nullptr, 0};
        bool filtered = false;
        if (request.enable_bitset_filter_ && request.bitset_filter_ != nullptr && !request.bitset_filter_->Words().empty()) {
            f.invalid_label_bits = request.bitset_filter_->Words().data();
            f.n_label_bits = request.bitset_filter_->Words().size() * 64;
            filtered = true;
        }
        if (request.enable_filter_ && request.filter_) {
            deny.assign((labels_host_.size() + 31) / 32, 0);
            for (size_t i = 0; i < labels_host_.size(); ++i) {
                if (!request.filter_(labels_host_[i])) {
                    deny[i >> 5] |= 1u << (i & 31);
                }
            }
            f.deny_inner_bits = deny.data();
            f.n_inner_bits = labels_host_.size();
            filtered = true;
        }
        const vb200_filter* fp = filtered ? &f : nullptr;
        if (request.mode_ == SearchMode::RANGE_SEARCH) {
            return range_impl(request.query_, request.radius_, request.params_str_, request.limited_size_, fp);
        }
        return knn_impl(request.query_, request.topk_, request.params_str_, fp);
    }

    Expected<DatasetPtr>
    range_impl(const DatasetPtr& query, float radius, const std::string& parameters, int64_t limited_size,
               const vb200_filter* filter) const {
        return safe_call<DatasetPtr>([&]() {
            return range_over_knn([&](int64_t k, const vb200_filter* f) { return knn_impl(query, k, parameters, f); },
                                  query, GetNumElements(), radius, 0.0f, limited_size, filter, labels_host_);
        });
    }

    Expected<void>
    Serialize(std::ostream& out) const override {
        return safe_void([&]() {
            std::lock_guard<std::mutex> lock(mu_);
            write_header(out, file_header());
            const uint64_t n_total = labels_host_.size();
            write_pod<uint64_t>(out, n_total);
            if (n_total > 0) {
                // fp32 rows or bf16 bit patterns, as stored
                std::vector<uint8_t> rows(n_total * dim_ * (quant_ == VB200_QUANT_FP32 ? 4 : 2));
                check_status(vb200_bf_get_rows(handle_, rows.data()));
                write_array(out, rows);
                write_array(out, labels_host_);
            }
            write_array(out, removed_labels_);
            check_stream_written(out);
        });
    }

    Expected<void>
    Deserialize(std::istream& in) override {
        return safe_void([&]() {
            std::lock_guard<std::mutex> lock(mu_);
            if (!labels_host_.empty()) {
                fail(ErrorType::INDEX_NOT_EMPTY, "failed to Deserialize: index is not empty");
            }
            read_header(in, file_header());
            const uint64_t n_total = read_pod<uint64_t>(in);
            if (n_total > 0) {
                auto rows = read_array<uint8_t>(in, n_total * dim_ * (quant_ == VB200_QUANT_FP32 ? 4 : 2), "rows");
                auto labels = read_array<int64_t>(in, n_total, "labels");
                check_status(vb200_bf_set_rows(handle_, rows.data(), n_total, labels.data()));
                labels_host_ = std::move(labels);
            }
            auto removed = read_array_any<int64_t>(in, "removed labels");
            check_end_mark(in);
            if (!removed.empty()) {
                check_status(remove_labels(removed.data(), removed.size(), nullptr));
                removed_labels_ = std::move(removed);
            }
        });
    }

    Expected<DatasetPtr>
    knn_impl(const DatasetPtr& query, int64_t k, const std::string& parameters, const vb200_filter* filter) const {
        if (k <= KNN_PAGE || query == nullptr || query->GetNumElements() == 0 || vb200_bf_num_elements(handle_) == 0) {
            return knn_page(query, k, parameters, filter);
        }
        return safe_call<DatasetPtr>([&]() {
            check_base(query, dim_, false);
            return knn_in_pages([&](const DatasetPtr& one, int64_t kk, const vb200_filter* f, int64_t) {
                return knn_page(one, kk, parameters, f);
            }, query, dim_, k, filter, labels_host_);
        });
    }

    Expected<DatasetPtr>
    knn_page(const DatasetPtr& query, int64_t k, const std::string& parameters, const vb200_filter* filter) const {
        return safe_call<DatasetPtr>([&]() {
            check_argument(query != nullptr, "query is null");
            check_argument(k > 0, "k must be greater than 0");
            if (!parameters.empty()) {
                Json root = Json::Parse(parameters);  // "{}", {"parallelism": n} or nested (bruteforce_parameter.h:44-78)
                check_argument(root.IsObject(), "search parameters must be a JSON object");
            }
            if (query->GetNumElements() == 0 || vb200_bf_num_elements(handle_) == 0) {
                return make_empty_result();
            }
            check_base(query, dim_, false);
            const int64_t nq = query->GetNumElements();
            auto* ids = new int64_t[static_cast<size_t>(nq * k)];
            auto* dists = new float[static_cast<size_t>(nq * k)];
            int status = vb200_bf_search_filtered(handle_, query->GetFloat32Vectors(), nq, static_cast<uint32_t>(k),
                                                  filter, ids, dists);
            if (status != 0) {
                delete[] ids;
                delete[] dists;
                check_status(status);
            }
            std::string stats = "{\"dist_cmp\":" + std::to_string(vb200_bf_num_elements(handle_) * nq) + "}";
            return pack_result(ids, dists, nq, k, stats);
        });
    }

    int64_t GetNumElements() const override { return vb200_bf_num_elements(handle_); }
    int64_t GetMemoryUsage() const override {
        return vb200_bf_num_elements(handle_) * dim_ * (quant_ == VB200_QUANT_FP32 ? 4 : 2);
    }
    std::string GetIndexType() const override { return "brute_force"; }

private:
    void
    add_locked(const DatasetPtr& base) {
        check_argument(base != nullptr, "dataset is null");
        if (base->GetNumElements() == 0) {
            return;
        }
        if (base->GetFloat32Vectors() == nullptr && base->GetFloat16Vectors() != nullptr &&
            quant_ == VB200_QUANT_BF16) {
            // rows that are already bf16 bit patterns (Dataset::Float16Vectors, dataset.h:277-284)
            check_argument(base->GetDim() == static_cast<int64_t>(dim_) && base->GetIds() != nullptr,
                           "dataset does not match the index");
            check_status(vb200_bf_add_bf16(handle_, base->GetFloat16Vectors(),
                                           static_cast<uint64_t>(base->GetNumElements()), base->GetIds()));
            labels_host_.insert(labels_host_.end(), base->GetIds(), base->GetIds() + base->GetNumElements());
            return;
        }
        check_base(base, dim_, true);
        check_status(vb200_bf_add(handle_, base->GetFloat32Vectors(), static_cast<uint64_t>(base->GetNumElements()),
                                  base->GetIds()));
        labels_host_.insert(labels_host_.end(), base->GetIds(), base->GetIds() + base->GetNumElements());
    }

    int
    remove_labels(const int64_t* ids, uint64_t count, uint64_t* removed) {
        return vb200_bf_remove(handle_, ids, count, removed);
    }

    FileHeader
    file_header() const {
        return FileHeader{FILE_KIND_BRUTE_FORCE, dim_, 0u, 0u, metric_, quant_};
    }

    std::vector<int64_t> labels_host_;     // ids in insertion order, for callback filters
    std::vector<int64_t> removed_labels_;  // every id Remove was asked for, replayed after a reload

    uint32_t dim_;
    int metric_;
    int quant_ = VB200_QUANT_FP32;
    vb200_bf_t handle_ = nullptr;
    mutable std::mutex mu_;
};

}  // namespace

Expected<std::shared_ptr<Index>>
Factory::CreateIndex(const std::string& name, const std::string& parameters) {
    return safe_call<std::shared_ptr<Index>>([&]() -> std::shared_ptr<Index> {
        std::string lowered = lower(name);  // names are case-insensitive (src/factory/index_registry.cpp:41-47)
        if (lowered != "ivf" && lowered != "brute_force") {
            fail(ErrorType::UNSUPPORTED_INDEX, "failed to create index(unsupported): " + name);
        }
        CommonParam common = parse_common(parameters);
        if (lowered == "ivf") {
            return std::make_shared<GpuIVF>(common);
        }
        return std::make_shared<GpuBruteForce>(common);
    });
}

}  // namespace vsag
