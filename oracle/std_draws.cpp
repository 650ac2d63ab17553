// Test infrastructure only.  The C++ library's own generator and distributions, as
// KMeansCluster::select_initial_centroids_kmeans_plus_plus uses them (kmeans_cluster.cpp:388-417),
// exported so a test can hold the C restatement of those draws (vsag_oracle.c: orc_std_draws)
// against the real thing.
#include <cstdint>
#include <random>

extern "C" __attribute__((visibility("default"))) void
std_draws(uint32_t seed, uint64_t n, uint64_t count, uint64_t* ints, double* reals) {
    std::mt19937 gen(seed);
    for (uint64_t i = 0; i < count; ++i) {
        std::uniform_int_distribution<uint64_t> dis(0, n - 1);
        ints[i] = dis(gen);
        std::uniform_real_distribution<double> prob(0.0, static_cast<double>(i + 1) * 1.5);
        reals[i] = prob(gen);
    }
}
