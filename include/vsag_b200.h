/*
 * vsag_b200.h -- C ABI of the B200 (sm_100a) engine for VSAG's dense data-parallel hot path:
 * IVF partition training (k-means), SQ8 / 1-bit RaBitQ encoders, the IVF inverted-list scan with
 * fused top-k and fp32 rerank, and exact BruteForce kNN.
 *
 * This is the boundary a VSAG build binds to replace its CPU implementation of that path.  Each
 * entry point names the reference interface it stands in for (paths are relative to the
 * antgroup/vsag source tree).
 *
 * Conventions
 *   - Every function returns 0 on success or a negative VB200_* code (same numbering as
 *     include/vsag/vsag_c_api.h:20-34, so a caller can forward it as an Error_t code).  The text of
 *     the last error of the calling thread is read with vb200_last_error().
 *   - Matrices are row-major and dense.  Data pointers may be host or device pointers; the library
 *     detects which (cudaPointerGetAttributes), stages host data through the current stream, and
 *     returns after the results are complete in the caller's memory.  Pointers are borrowed for
 *     the duration of the call only.
 *   - Handles own device memory and are bound to the CUDA device current at creation.
 *   - There is no CPU fallback: without a CUDA device every compute entry point fails with
 *     VB200_INTERNAL_ERROR.
 */
#ifndef VSAG_B200_H_
#define VSAG_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define VB200_API __attribute__((visibility("default")))
#else
#define VB200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define VB200_SUCCESS 0
#define VB200_UNKNOWN_ERROR -1
#define VB200_INTERNAL_ERROR -2
#define VB200_INVALID_ARGUMENT -3
#define VB200_WRONG_STATUS -4
#define VB200_BUILD_TWICE -5
#define VB200_INDEX_NOT_EMPTY -6
#define VB200_UNSUPPORTED_INDEX -7
#define VB200_UNSUPPORTED_INDEX_OPERATION -8
#define VB200_DIMENSION_NOT_EQUAL -9
#define VB200_INDEX_EMPTY -10
#define VB200_NO_ENOUGH_MEMORY -11

/* metric_type values of IndexCommonParam (src/index_common_param.cpp:117-174). */
#define VB200_METRIC_L2 0
#define VB200_METRIC_IP 1
#define VB200_METRIC_COSINE 2

/* base_quantization_type values served by the engine (src/algorithm/ivf/ivf.cpp:140-395). */
#define VB200_QUANT_FP32 0
#define VB200_QUANT_SQ8 1
#define VB200_QUANT_RABITQ 2
#define VB200_QUANT_BF16 3
#define VB200_QUANT_FP16 4   /* IVF buckets only */
#define VB200_QUANT_SQ8_UNIFORM 5   /* IVF buckets only */

/* SQTrainMode (src/quantization/scalar_quantization/scalar_quantization_trainer.h:25-29). */
#define VB200_SQ_TRAIN_CLASSIC 1
#define VB200_SQ_TRAIN_TRUNC_BOUND 3

typedef struct vb200_ivf* vb200_ivf_t;
typedef struct vb200_bf* vb200_bf_t;
typedef struct vb200_comm* vb200_comm_t;

/* ---------------------------------------------------------------------------------------------
 * Library state
 * ------------------------------------------------------------------------------------------- */

/* Copies the calling thread's last error text into buf (NUL terminated) and returns its code. */
VB200_API int vb200_last_error(char* buf, size_t buf_len);

/* vb200_kmeans_train keeps its device workspace between calls (allocating it costs more than the iterations it
 * serves); this frees it.  Indexes own their workspaces and free them with the handle. */
VB200_API int vb200_release_workspaces(void);

/* CUDA stream (a cudaStream_t) the calling thread's subsequent calls launch on; NULL = the
 * default stream. */
VB200_API int vb200_set_stream(void* cuda_stream);

/* Number of kernels this library has launched in the process so far. */
VB200_API uint64_t vb200_kernel_launches(void);

/* Chooses how the dense contractions (k-means assignment, routing, BruteForce) nominate
 * candidates: 1 (default) = tcgen05 tensor-core kernels, 0 = the fixed-order fp32 SIMT kernels.
 * Either way the survivors are re-scored in the reference's exact operation order, so results are
 * the same; the switch exists for cross-checking and timing.  The environment variable
 * VB200_DISABLE_TC=1 sets the initial value to 0. */
VB200_API int vb200_set_tensor_cores(int enable);

/* Test hook with no counterpart in the reference.  Every wait inside the tensor-core kernels (on a
 * copy, on an accumulator) polls a bounded number of times; when a wait runs out the kernel stops
 * taking work, frees its tensor memory and returns, and the call fails with VB200_INTERNAL_ERROR
 * while the CUDA context stays usable.  This sets that number of polls (a negative value restores
 * the default, 2^24; 0 makes every wait give up at once) so that a test can make a wait run out on
 * purpose and watch the error path. */
VB200_API int vb200_debug_set_wait_limit(int32_t polls);

/* Number of CUDA devices visible, or a negative VB200_* code. */
VB200_API int vb200_device_count(void);

/* ---------------------------------------------------------------------------------------------
 * SQ8 scalar quantizer
 * ------------------------------------------------------------------------------------------- */

/* Per-dimension bounds.  Replaces ScalarQuantizer<metric,8>::TrainImpl
 * (src/quantization/scalar_quantization/scalar_quantizer.cpp:51-74) and
 * ScalarQuantizationTrainer::Train (scalar_quantization_trainer.cpp:31-146): at most 100000 rows
 * sampled as row (j * (2147483647 % n)) % n, then CLASSIC min/max or TRUNC_BOUND order
 * statistics.  Outputs lower[dim] and diff[dim] = upper - lower, bit-equal to the reference for
 * finite inputs. */
VB200_API int vb200_sq8_train(const float* data, uint64_t count, uint32_t dim, int mode, float* lower, float* diff);

/* codes[count x dim], one byte per dimension.  Replaces ScalarQuantizer<metric,8>::EncodeOneImpl /
 * EncodeBatch (scalar_quantizer.cpp:85-110); bit-exact. */
VB200_API int vb200_sq8_encode(const float* data, uint64_t count, uint32_t dim, const float* lower,
                     const float* diff, uint8_t* codes);

/* ---------------------------------------------------------------------------------------------
 * k-means (IVF partition training)
 * ------------------------------------------------------------------------------------------- */

/* labels[i] = argmin_j |c_j|^2 - 2<c_j, x_i>, lowest j on ties; *mean_err (optional) = mean of
 * (min + |x_i|^2).  Replaces KMeansCluster::find_nearest_one_with_blas
 * (src/impl/cluster/kmeans_cluster.cpp:192-305) for every k (the reference switches to an
 * approximate graph search at k >= 10000, :307-365). */
VB200_API int vb200_kmeans_assign(const float* data, uint64_t count, uint32_t dim, const float* centroids,
                        uint32_t k, int32_t* labels, double* mean_err);

/* One centroid update from labels: mean of the members, empty clusters re-seeded from data row
 * (j * 2654435761 + iter) % count.  Replaces kmeans_cluster.cpp:106-172.  centroids[k x dim] is
 * overwritten, counts[k] (optional) receives the cluster sizes. */
VB200_API int vb200_kmeans_update(const float* data, uint64_t count, uint32_t dim, const int32_t* labels,
                        uint32_t k, uint32_t iter, float* centroids, int32_t* counts);

/* `iters` Lloyd iterations starting from centroids[k x dim] (in/out).  Replaces
 * KMeansCluster::Run (kmeans_cluster.cpp:46-190) with caller-supplied initial centroids.
 * labels[count] (optional) receives the labels of the last assignment. */
VB200_API int vb200_kmeans_train(const float* data, uint64_t count, uint32_t dim, uint32_t k, int iters,
                       float* centroids, int32_t* labels, double* mean_err);

/* k-means++ seeding: centroids[k x dim] = k rows of data drawn as
 * KMeansCluster::select_initial_centroids_kmeans_plus_plus does (kmeans_cluster.cpp:383-435): the
 * first uniformly, each later one with probability proportional to its squared distance from the
 * nearest centre chosen so far.  The draws come from std::mt19937(seed) through the same standard
 * distributions; the reference seeds that generator from std::random_device (kmeans_cluster.cpp:75),
 * here the caller does.  picked[k] (optional) receives the chosen row numbers. */
VB200_API int vb200_kmeans_init(const float* data, uint64_t count, uint32_t dim, uint32_t k, uint32_t seed,
                      float* centroids, int64_t* picked);

/* Same labels as vb200_kmeans_assign, for callers that must not allocate.  No counterpart in the
 * reference: it exists for hosts where reaching the CUDA allocator is not an option (a serving
 * thread with a fixed device-memory budget, or one that cannot take the device-wide
 * synchronisation an allocation or free implies).  It calls no cudaMalloc/cudaFree and no
 * allocating library routine; the one piece of scratch it needs, the centroid norms, sits in a
 * fixed 256 KiB array inside the library, so k is limited to 65536 (larger k fails with
 * VB200_INVALID_ARGUMENT).  data, centroids and labels must be device pointers.
 * The first call on each device looks up the array's device address; make that first call before
 * any stream capture.  All calls share the array (it keeps the previous call's contents, which the
 * next call overwrites before use), so two calls that overlap on the same GPU race: serialise
 * them. */
VB200_API int vb200_kmeans_assign_noalloc(const float* data_dev, uint64_t count, uint32_t dim,
                                const float* centroids_dev, uint32_t k, int32_t* labels_dev);

/* ---------------------------------------------------------------------------------------------
 * RaBitQ, 1 bit per dimension, fp32 query ("standard" layout)
 * ------------------------------------------------------------------------------------------- */

/* Bytes per code record: ceil(dim/8) sign bytes padded to 4, fp32 norm, fp32 error
 * (src/quantization/rabitq_quantization/rabitq_quantizer.cpp:102-185). */
VB200_API uint64_t vb200_rabitq_code_size(uint32_t dim);

/* centroid[dim] = rotation * mean(data).  Replaces RaBitQuantizer::TrainImpl
 * (rabitq_quantizer.cpp:209-254); `rotation` is the dim x dim row-major orthogonal matrix the
 * reference draws in RandomOrthogonalMatrix::Train
 * (src/impl/transform/random_orthogonal_transformer.cpp:32-149). */
VB200_API int vb200_rabitq_train(const float* data, uint64_t count, uint32_t dim, const float* rotation,
                       float* centroid);

/* codes[count x code_size].  Replaces RaBitQuantizer::EncodeOneInternal, 1-bit branch
 * (rabitq_quantizer.cpp:723-857). */
VB200_API int vb200_rabitq_encode(const float* data, uint64_t count, uint32_t dim, const float* rotation,
                        const float* centroid, uint8_t* codes);

/* out[count x (dim+1)]: rotated, centred, normalised query followed by its norm.  Replaces
 * RaBitQuantizer::ProcessQueryImpl (rabitq_quantizer.cpp:2130-2217). */
VB200_API int vb200_rabitq_process_query(const float* queries, uint64_t count, uint32_t dim,
                               const float* rotation, const float* centroid, float* out);

/* ---------------------------------------------------------------------------------------------
 * IVF index (vsag::Factory::CreateIndex("ivf", ...))
 * ------------------------------------------------------------------------------------------- */

/* Replaces IVF::IVF (src/algorithm/ivf/ivf.cpp:412-474): nlist = buckets_count, quant =
 * base_quantization_type (VB200_QUANT_FP32, the reference's default, VB200_QUANT_SQ8, VB200_QUANT_RABITQ, or the
 * half-precision codecs VB200_QUANT_BF16 / VB200_QUANT_FP16 of
 * src/quantization/scalar_quantization/half_precision_quantizer.cpp:54-123),
 * use_reorder keeps the fp32 rows for exact rerank (precise_quantization_type fp32). */
VB200_API int vb200_ivf_create(uint32_t dim, int metric, uint32_t nlist, int quant, int use_reorder,
                     vb200_ivf_t* out);
VB200_API int vb200_ivf_destroy(vb200_ivf_t index);

/* List sharding for multi-GPU search: this handle keeps only lists l with l % world == rank.
 * Must be called before the first add.  Default: rank 0 of 1. */
VB200_API int vb200_ivf_set_shard(vb200_ivf_t index, uint32_t rank, uint32_t world);

/* IVF::Train (ivf.cpp:564-588): k-means on the rows given (the caller has already sampled them;
 * the reference samples with std::random_device, src/utils/util_functions.cpp:273-330), initial
 * centroids = init[nlist x dim] or the first nlist rows when init is NULL; then trains the
 * bucket quantizer on the same rows.  For RABITQ, `rotation` must have been set first. */
VB200_API int vb200_ivf_train(vb200_ivf_t index, const float* data, uint64_t count, int kmeans_iters,
                    const float* init);

/* use_residual (IVF creation parameter; sq8 buckets): lists hold the codes of x - centroid; the quantizer is
 * trained on the residuals of the training rows (BucketDataCell::Train, src/datacell/bucket_datacell.h:593-614),
 * a row's L2 bias -2 * IP(c, decoded) - IP(c, c) is kept beside its code (:621-651) and a distance is the
 * quantizer's distance between the raw query and the residual code, minus the bias (L2), minus 2 * IP(q, c)
 * (L2) or IP(q, c) (IP / cosine) (:552-566).  Choose before training.  Such an index scans without list pruning. */
VB200_API int vb200_ivf_set_use_residual(vb200_ivf_t index, int use_residual);

/* buckets_per_data (IVF creation parameter, src/algorithm/ivf/ivf.cpp:607, :659-676): every vector is stored
 * in that many of its nearest lists; a search looks for buckets_per_data times as many postings and folds the
 * duplicates of a vector into its smallest distance (:1722-1727, :1799-1825).  Set before the first add; 1 is
 * the default; not available on a sharded index.  With it, vb200_ivf_add's labels_in (when given) holds
 * count x buckets_per_data list ids, vector by vector. */
VB200_API int vb200_ivf_set_buckets_per_data(vb200_ivf_t index, uint32_t buckets_per_data);

/* SQ8 uniform (base_quantization_type "sq8_uniform", SQ8UniformQuantizer,
 * src/quantization/scalar_quantization/sq8_uniform_quantizer.cpp:76-186): one lower bound and one range for all
 * dimensions; codes carry their uint64 squared norm (L2) or fp32 value sum (IP / cosine), queries are encoded
 * like rows and distances come from the exact integer inner product of the byte codes. */
VB200_API int vb200_ivf_set_sq8_uniform_model(vb200_ivf_t index, float lower, float diff);
VB200_API int vb200_ivf_get_sq8_uniform_model(vb200_ivf_t index, float* lower, float* diff);

/* Model import/export, the pieces IVF::ExportModel / Serialize carry (ivf.cpp:990-1056,
 * :1677-1691): centroids[nlist x dim]; SQ8 lower[dim], diff[dim]
 * (scalar_quantizer.cpp:199-204); RaBitQ rotation[dim x dim], centroid[dim]
 * (rabitq_quantizer.cpp:2245-2254). */
VB200_API int vb200_ivf_set_centroids(vb200_ivf_t index, const float* centroids);
VB200_API int vb200_ivf_get_centroids(vb200_ivf_t index, float* centroids);
VB200_API int vb200_ivf_set_sq8_model(vb200_ivf_t index, const float* lower, const float* diff);
VB200_API int vb200_ivf_get_sq8_model(vb200_ivf_t index, float* lower, float* diff);
VB200_API int vb200_ivf_set_rabitq_rotation(vb200_ivf_t index, const float* rotation);
VB200_API int vb200_ivf_set_rabitq_centroid(vb200_ivf_t index, const float* centroid);
VB200_API int vb200_ivf_get_rabitq_centroid(vb200_ivf_t index, float* centroid);

/* IVF::Add (ivf.cpp:590-724): assigns each row to its nearest centroid (exact, where the
 * reference asks an approximate graph router), encodes it and appends it to that list in row
 * order.  labels_in (optional) supplies the list of every row instead of computing it.
 * ids[count] are the user labels; inner ids continue from the current element count. */
VB200_API int vb200_ivf_add(vb200_ivf_t index, const float* data, uint64_t count, const int64_t* ids,
                  const int32_t* labels_in);

/* Number of vectors added (all shards count every row) and bytes of device memory held. */
VB200_API int64_t vb200_ivf_num_elements(vb200_ivf_t index);
VB200_API int64_t vb200_ivf_memory_usage(vb200_ivf_t index);

/* Inverted-file layout readback for parity checks: list_sizes[nlist]; then, with offsets the
 * exclusive prefix of the sizes, codes[total x code_size] and inner_ids[total] in list order
 * (the layout of BucketDataCell, src/datacell/bucket_datacell.h:891-904).  Any pointer may be
 * NULL.  code_size = dim (SQ8) or vb200_rabitq_code_size(dim). */
VB200_API int vb200_ivf_get_lists(vb200_ivf_t index, int64_t* list_sizes, uint8_t* codes, int64_t* inner_ids);

/* The inverse of vb200_ivf_get_lists: fills an empty, trained index (centroids and quantizer model
 * set, e.g. with the setters above) from lists that are already encoded, in the layout IVF::Serialize
 * writes for its bucket datacell (src/datacell/bucket_datacell.h:891-904: per list its codes, its
 * inner ids, its size) plus the label table (ivf.cpp:997).  list_sizes[nlist] is host memory;
 * codes[total x code_size], inner_ids[total], labels[n_total] (user label of every inner id) and
 * rows[n_total x dim] (the fp32 vectors by inner id as vb200_ivf_get_rows returns them; required when
 * reorder is on, else may be NULL) may be host or device memory.  A shard keeps only its own lists
 * (list % world == rank).  Nothing is re-encoded or normalised again: a search on the loaded index
 * returns what it returned on the index the lists came from. */
VB200_API int vb200_ivf_set_lists(vb200_ivf_t index, const int64_t* list_sizes, const uint8_t* codes,
                        const int64_t* inner_ids, const int64_t* labels, uint64_t n_total,
                        const float* rows);

/* The fp32 rows an index with reorder keeps for the rerank (the reference's reorder codes,
 * ivf.cpp:999-1005), [num vectors ever added x dim] by inner id, normalised when the metric is cosine;
 * rows may be host or device memory. */
VB200_API int vb200_ivf_get_rows(vb200_ivf_t index, float* rows);

/* IVF::KnnSearch / SearchWithRequest batch branch (ivf.cpp:892-907, :2052-2354, :1693-1828):
 * for each of nq queries, routes to the nprobe = scan_buckets_count nearest lists (exact),
 * scans them, keeps the k best (factor*k when reorder is on, then reranks with the fp32 rows,
 * src/impl/reorder/flatten_reorder.cpp:76-118).  ids[nq x k] user labels (-1 pad),
 * dists[nq x k] ascending (+inf pad).
 * bucket_ids (optional, [nq x nprobe], -1 = skip) bypasses routing like
 * SearchRequest::bucket_ids_ (include/vsag/search_request.h:227). */
VB200_API int vb200_ivf_search(vb200_ivf_t index, const float* queries, uint64_t nq, uint32_t k,
                     uint32_t nprobe, float factor, const int32_t* bucket_ids, int64_t* ids,
                     float* dists);

/* Id filter of a search (SearchRequest filters, include/vsag/search_request.h; BlackListFilter,
 * src/impl/filter/black_list_filter.cpp:25-31).  Both parts are optional; pointers may be host or
 * device memory.
 *   invalid_label_bits: the reference's bitset filter, bit (label & 0xFFFFFFFF) set = filtered out;
 *                       labels beyond n_label_bits pass.
 *   deny_inner_bits:    bit i set = the i-th vector ever added (inner id i) is filtered out; this
 *                       is what a host callback filter is materialised into. */
typedef struct vb200_filter {
    const uint64_t* invalid_label_bits;
    uint64_t n_label_bits;
    const uint32_t* deny_inner_bits;
    uint64_t n_inner_bits;
} vb200_filter;

/* vb200_ivf_search with an id filter (and always without the vectors removed so far). */
VB200_API int vb200_ivf_search_filtered(vb200_ivf_t index, const float* queries, uint64_t nq, uint32_t k,
                              uint32_t nprobe, float factor, const int32_t* bucket_ids,
                              const vb200_filter* filter, int64_t* ids, float* dists);

/* Index::Remove with RemoveMode::MARK_REMOVE (include/vsag/index.h:186-200): the vectors with these
 * labels stay in their lists but no search returns them any more.  removed (optional) receives how
 * many labels were found and newly marked. */
VB200_API int vb200_ivf_remove(vb200_ivf_t index, const int64_t* labels, uint64_t count, uint64_t* removed);

/* Routing only, like the disable_bucket_scan search mode (IVF::route_buckets_only,
 * ivf.cpp:1589-1660): bucket_ids[nq x nprobe] ascending by centroid distance,
 * bucket_dists optional. */
VB200_API int vb200_ivf_route(vb200_ivf_t index, const float* queries, uint64_t nq, uint32_t nprobe,
                    int32_t* bucket_ids, float* bucket_dists);

/* Per-call search options of IndexSearchParameter (src/algorithm/index_search_parameter.h:27-57).
 * enable_reorder = 0: an index built with use_reorder answers with the quantized distances of its k best
 * (no factor * k candidates, no exact re-ranking: IVF::SearchWithRequest, src/algorithm/ivf/ivf.cpp:2312-2321).
 * has_timeout != 0: once timeout_ms have passed since the call's device work began the scan hands out no
 * further list, the call returns what it found and *timed_out is 1 -- the reference checks its timer between
 * buckets and reports is_timeout in the statistics (ivf.cpp:1747-1751). */
typedef struct vb200_search_options {
    int enable_reorder;
    int has_timeout;
    double timeout_ms;
} vb200_search_options;

/* vb200_ivf_search_filtered with options (NULL = defaults: reorder on, no timeout); timed_out may be NULL. */
VB200_API int vb200_ivf_search_ex(vb200_ivf_t index, const float* queries, uint64_t nq, uint32_t k, uint32_t nprobe,
                        float factor, const int32_t* bucket_ids, const vb200_filter* filter,
                        const vb200_search_options* options, int64_t* ids, float* dists, int* timed_out);

/* Called by vb200_ivf_search_partial between its two scan phases: bounds_dev[nq] holds, per query,
 * the distance bound this shard has found so far (+inf = none).  The callee replaces every entry
 * by the minimum over all shards (an all-reduce with MIN on the communicator it owns), enqueued
 * on, or ordered with, cuda_stream; it returns 0 on success. */
typedef int (*vb200_exchange_fn)(float* bounds_dev, uint64_t nq, void* cuda_stream, void* arg);

/* Same search, but stops before the label translation and returns this shard's partial result as
 * device-resident sortable keys for a cross-GPU merge: keys_dev[nq x k] (uint64, distance in the
 * high word) and labels_dev[nq x k] must be device pointers.  bucket_ids (optional, as in
 * vb200_ivf_search) lets the ranks route disjoint slices of the batch and share the lists.
 * exchange (optional) shares the per-query bounds between the shards after each has scanned the
 * nearest list it holds; without it every shard prunes with its own bounds only. */
VB200_API int vb200_ivf_search_partial(vb200_ivf_t index, const float* queries, uint64_t nq, uint32_t k,
                             uint32_t nprobe, float factor, const int32_t* bucket_ids,
                             vb200_exchange_fn exchange, void* exchange_arg, uint64_t* keys_dev,
                             int64_t* labels_dev);

/* Logical bytes of codes the last search scanned (sum over queries of probed list lengths x
 * code size), the figure the HBM roofline of the scan is computed from. */
VB200_API int64_t vb200_ivf_last_scan_bytes(vb200_ivf_t index);

/* Bytes of codes the last search actually read after list pruning: an SQ8 scan drops a (query,
 * list) pair unscanned when the triangle inequality on the list's radius shows that nothing in the
 * list can beat the query's current k-th candidate.  The result is the same as without pruning. */
VB200_API int64_t vb200_ivf_last_scanned_bytes(vb200_ivf_t index);

/* Turns that list pruning off (0) or on (non-zero, the default); for cross-checks. */
VB200_API int vb200_ivf_set_list_pruning(vb200_ivf_t index, int enable);

/* Device time of the last search's list-scan kernel in milliseconds, from CUDA events recorded
 * around its launch on the stream it ran on. */
VB200_API int vb200_ivf_last_scan_ms(vb200_ivf_t index, float* ms);

/* Merges `parts` partial results laid out [parts][nq][k] (as gathered from the ranks) into
 * ids[nq x k], dists[nq x k].  Inputs are device pointers; outputs host or device. */
VB200_API int vb200_merge_partials(const uint64_t* keys_dev, const int64_t* labels_dev, uint32_t parts,
                         uint64_t nq, uint32_t k, int64_t* ids, float* dists);

/* ---------------------------------------------------------------------------------------------
 * BruteForce index (vsag::Factory::CreateIndex("brute_force", ...))
 * ------------------------------------------------------------------------------------------- */

/* Replaces BruteForce::BruteForce with base_quantization_type fp32 or bf16
 * (src/algorithm/bruteforce/bruteforce.cpp:1273-1361). */
VB200_API int vb200_bf_create(uint32_t dim, int metric, int quant, vb200_bf_t* out);
VB200_API int vb200_bf_destroy(vb200_bf_t index);

/* BruteForce::Add (bruteforce.cpp:213-293): fp32 rows; a bf16 index rounds them with
 * generic::FloatToBF16 (src/simd/generic.cpp:198-202). */
VB200_API int vb200_bf_add(vb200_bf_t index, const float* data, uint64_t count, const int64_t* ids);

/* Rows that are already bf16 (uint16 bit patterns), for bf16 indexes only. */
VB200_API int vb200_bf_add_bf16(vb200_bf_t index, const uint16_t* data, uint64_t count, const int64_t* ids);

/* The rows as the index stores them (what BruteForce::Serialize writes as inner_codes_,
 * src/algorithm/bruteforce/bruteforce.cpp:685-693): fp32 [n x dim], or bf16 bit patterns [n x dim] for a bf16 index,
 * normalised when the metric is cosine; n counts every vector ever added.  vb200_bf_set_rows puts
 * such rows back into an empty index without normalising or rounding them again.  Pointers may be
 * host or device memory. */
VB200_API int vb200_bf_get_rows(vb200_bf_t index, void* rows);
VB200_API int vb200_bf_set_rows(vb200_bf_t index, const void* rows, uint64_t count, const int64_t* ids);

VB200_API int64_t vb200_bf_num_elements(vb200_bf_t index);

/* BruteForce::KnnSearch (bruteforce.cpp:354-635) for a batch of nq queries (the reference takes
 * one query per call; nq = 1 gives the same result).  ids[nq x k] labels (-1 pad),
 * dists[nq x k] ascending (+inf pad). */
VB200_API int vb200_bf_search(vb200_bf_t index, const float* queries, uint64_t nq, uint32_t k, int64_t* ids,
                    float* dists);

/* vb200_bf_search with an id filter, and Index::Remove(MARK_REMOVE); see vb200_ivf_search_filtered and
 * vb200_ivf_remove. */
VB200_API int vb200_bf_search_filtered(vb200_bf_t index, const float* queries, uint64_t nq, uint32_t k,
                             const vb200_filter* filter, int64_t* ids, float* dists);
VB200_API int vb200_bf_remove(vb200_bf_t index, const int64_t* labels, uint64_t count, uint64_t* removed);

/* Partial result for a row-sharded index, see vb200_ivf_search_partial. */
VB200_API int vb200_bf_search_partial(vb200_bf_t index, const float* queries, uint64_t nq, uint32_t k,
                            uint64_t* keys_dev, int64_t* labels_dev);

/* ---------------------------------------------------------------------------------------------
 * Sharded search over the GPUs of one node: one process per GPU, lists (IVF) or rows (BruteForce)
 * dealt to the ranks, one exchange step.  The reference's analogue is a set of shard indexes built
 * from one model whose results the caller merges (IVF::Merge and the model-equality checks,
 * src/algorithm/ivf/ivf.cpp:1989-2050); here the exchange runs over NVLink through NCCL, which the
 * library opens itself (libnccl.so.2) when the first communicator is created.
 * ------------------------------------------------------------------------------------------- */
#define VB200_COMM_ID_BYTES 128

/* Rank 0 draws the communicator's id and hands it to the other ranks by whatever means the host has (a
 * file, a socket, an existing process group); then every rank calls vb200_comm_init with its rank, after
 * selecting its GPU with cudaSetDevice.  vb200_comm_init blocks until all `world` ranks have called it. */
VB200_API int vb200_comm_unique_id(uint8_t* id_out /* VB200_COMM_ID_BYTES */);
VB200_API int vb200_comm_init(vb200_comm_t* comm_out, const uint8_t* id, int rank, int world);
VB200_API int vb200_comm_destroy(vb200_comm_t comm);
VB200_API int vb200_comm_rank(vb200_comm_t comm);
VB200_API int vb200_comm_world(vb200_comm_t comm);

/* The whole search step of a list-sharded IVF index (vb200_ivf_set_shard(rank, world) on every rank, all
 * ranks holding the same centroids and quantizer model), called by all ranks with the same query batch:
 * each rank routes its slice of the batch, the probe lists and their centroid distances are all-gathered,
 * every rank scans the probed lists it owns -- first each query's nearest list, then, after an all-reduce
 * (MIN) of the per-query bounds, the rest -- and the per-rank top-k, packed as (key, label) arrays, are
 * all-gathered and merged on every rank.  Every rank receives the full result, equal to the unsharded
 * index's.  One host synchronisation at the end (plus the status checks of the tensor-core kernels). */
VB200_API int vb200_ivf_search_sharded(vb200_ivf_t index, vb200_comm_t comm, const float* queries, uint64_t nq,
                                       uint32_t k, uint32_t nprobe, float factor, int64_t* ids, float* dists);

/* The same for a row-sharded BruteForce index: every rank searches its rows for the whole batch, the
 * per-rank top-k are all-gathered and merged on every rank. */
VB200_API int vb200_bf_search_sharded(vb200_bf_t index, vb200_comm_t comm, const float* queries, uint64_t nq,
                                      uint32_t k, int64_t* ids, float* dists);

#ifdef __cplusplus
}
#endif

#endif /* VSAG_B200_H_ */
