// TEST INFRASTRUCTURE ONLY (checker + timed CPU baseline), never part of the product path.
//
// Thin extern "C" shim around the UNMODIFIED reference CPU implementation
// (src/PermutohedralLatticeCPU.h of MiguelMonteiro/permutohedral_lattice).  The header is
// included from where the reference tree lies (-I<reference>/src at build time); nothing of
// it is copied here.  Output: oracle/_ref/libpl_ref.so (git-ignored).
//
// Two things the header does not offer are obtained without editing it:
//  * access to the private hashTable / matrix members: `#define class struct` around the
//    include (the header never uses `class` inside template parameter lists);
//  * a hash table that never grows.  HashTableCPU::lookup (src/PermutohedralLatticeCPU.h:163-170)
//    computes h with the old capacity and lookupOffset (:59-62) may then double the capacity and
//    keep probing from that stale h, which creates a duplicate vertex per growth.  Replacing the
//    (public) arrays by larger ones of the constructor's own layout (:135-142) before filter()
//    keeps grow() from ever running, so size() is the number of distinct keys.
#include <cstdio>
#include <cmath>
#include <cstring>
#include <memory>
#include <vector>
#include <thread>
#include <chrono>

#define class struct
#include "PermutohedralLatticeCPU.h"
#undef class

namespace {

template <typename T>
struct RefRun {
    int n, pd, vd;
    PermutohedralLatticeCPU<T>* lattice;
    size_t capacity_before;
};

// Swap in a table of `capacity` slots laid out exactly as HashTableCPU's constructor does.
template <typename T>
void presize(PermutohedralLatticeCPU<T>& L, size_t capacity) {
    HashTableCPU<T>& t = L.hashTable;
    delete[] t.entries;
    delete[] t.keys;
    delete[] t.values;
    t.capacity = capacity;
    t.filled = 0;
    t.entries = new int[capacity];
    memset(t.entries, -1, capacity * sizeof(int));
    t.keys = new short[(size_t)t.pd * capacity / 2];
    t.values = new T[(size_t)t.vd * capacity / 2]();
}

size_t pow2_at_least(size_t x) {
    size_t c = 1 << 15;
    while (c < x) c <<= 1;
    return c;
}

// One PermutohedralLatticeCPU<T>(pd, vd, n).filter(out, in, pos, reverse)
// (src/LatticeFilterKernel.cpp:79-80).
template <typename T>
void* run_filter(T* out, const T* in, const T* positions, int n, int pd, int vd, int reverse,
                 long long min_vertices) {
    auto* L = new PermutohedralLatticeCPU<T>(pd, vd, n);
    if (min_vertices > 0) presize(*L, pow2_at_least(2 * (size_t)min_vertices + 8));
    size_t cap = L->hashTable.capacity;
    L->filter(out, in, positions, reverse != 0);
    if (min_vertices > 0 && L->hashTable.capacity != cap) {
        delete L;
        return nullptr;
    }
    return new RefRun<T>{n, pd, vd, L, cap};
}

template <typename T>
void get_matrix(void* h, int* vertex_out, T* weight_out) {
    auto* r = static_cast<RefRun<T>*>(h);
    size_t cnt = (size_t)r->n * (r->pd + 1);
    for (size_t i = 0; i < cnt; i++) {
        vertex_out[i] = r->lattice->matrix[i].offset / r->vd;
        weight_out[i] = r->lattice->matrix[i].weight;
    }
}

template <typename T>
void get_keys(void* h, short* keys_out) {
    auto* r = static_cast<RefRun<T>*>(h);
    size_t m = r->lattice->hashTable.size();
    memcpy(keys_out, r->lattice->hashTable.getKeys(), m * r->pd * sizeof(short));
}

template <typename T>
void free_run(void* h) {
    auto* r = static_cast<RefRun<T>*>(h);
    delete r->lattice;
    delete r;
}

// The per-batch-item loop of src/LatticeFilterKernel.cpp:152-179 (positions, then one fresh lattice
// per item), items dealt round-robin to `threads` std::threads (the reference itself is
// single-threaded; threads == 1 reproduces it).
template <typename T>
double run_batch(T* out, const T* in, const T* reference, int batch, int n, int n_in_channels,
                 int n_ref_channels, int n_sdims, const int* sdims, T spatial_std, T feature_std,
                 int reverse, long long min_vertices, int threads) {
    int pd = n_sdims + n_ref_channels, vd = n_in_channels + 1;
    if (threads < 1) threads = 1;
    std::vector<int> bad(threads, 0);
    auto t0 = std::chrono::steady_clock::now();
    auto work = [&](int tid) {
        std::vector<T> pos((size_t)n * pd);
        for (int b = tid; b < batch; b += threads) {
            const T* ref_b = reference ? reference + (size_t)b * n * n_ref_channels : nullptr;
            compute_kernel_cpu<T>(ref_b, pos.data(), n, n_ref_channels, n_sdims, sdims,
                                  spatial_std, feature_std);
            PermutohedralLatticeCPU<T> L(pd, vd, n);
            if (min_vertices > 0) presize(L, pow2_at_least(2 * (size_t)min_vertices + 8));
            size_t cap = L.hashTable.capacity;
            L.filter(out + (size_t)b * n * n_in_channels, in + (size_t)b * n * n_in_channels,
                     pos.data(), reverse != 0);
            if (min_vertices > 0 && L.hashTable.capacity != cap) bad[tid] = 1;
        }
    };
    std::vector<std::thread> pool;
    for (int t = 1; t < threads; t++) pool.emplace_back(work, t);
    work(0);
    for (auto& th : pool) th.join();
    auto t1 = std::chrono::steady_clock::now();
    for (int b : bad)
        if (b) return -1.0;
    return std::chrono::duration<double>(t1 - t0).count();
}

}  // namespace

extern "C" {

// src/PermutohedralLatticeCPU.h:452-474 (compute_kernel_cpu), called as
// src/LatticeFilterKernel.cpp:63 does.
void plref_compute_positions(const float* reference, float* positions, int n, int n_ref_channels,
                             int n_sdims, const int* sdims, float spatial_std, float feature_std) {
    compute_kernel_cpu<float>(reference, positions, n, n_ref_channels, n_sdims, sdims, spatial_std,
                              feature_std);
}
void plref_compute_positions_f64(const double* reference, double* positions, int n,
                                 int n_ref_channels, int n_sdims, const int* sdims,
                                 double spatial_std, double feature_std) {
    compute_kernel_cpu<double>(reference, positions, n, n_ref_channels, n_sdims, sdims, spatial_std,
                               feature_std);
}

// min_vertices == 0: table exactly as shipped (it grows, with the duplicate-vertex defect).
// min_vertices > 0: table pre-sized for that many vertices, and the call fails (returns NULL) if
// the table grew all the same.  Returns a handle for the structure queries below; free it with
// plref_free / plref_free_f64.
void* plref_filter(float* out, const float* in, const float* positions, int n, int pd, int vd,
                   int reverse, long long min_vertices) {
    return run_filter<float>(out, in, positions, n, pd, vd, reverse, min_vertices);
}
void* plref_filter_f64(double* out, const double* in, const double* positions, int n, int pd,
                       int vd, int reverse, long long min_vertices) {
    return run_filter<double>(out, in, positions, n, pd, vd, reverse, min_vertices);
}

int plref_num_vertices(void* h) { return static_cast<RefRun<float>*>(h)->lattice->hashTable.size(); }
int plref_num_vertices_f64(void* h) {
    return static_cast<RefRun<double>*>(h)->lattice->hashTable.size();
}

// 1 if the table kept its initial capacity during the run.
int plref_never_grew(void* h) {
    auto* r = static_cast<RefRun<float>*>(h);
    return r->lattice->hashTable.capacity == r->capacity_before;
}
int plref_never_grew_f64(void* h) {
    auto* r = static_cast<RefRun<double>*>(h);
    return r->lattice->hashTable.capacity == r->capacity_before;
}

// keys_out[M*pd]: vertex keys in creation order (hashTable.getKeys()).
void plref_keys(void* h, short* keys_out) { get_keys<float>(h, keys_out); }
void plref_keys_f64(void* h, short* keys_out) { get_keys<double>(h, keys_out); }

// Per pixel and remainder: vertex id (= matrix offset / vd) and barycentric weight
// (src/PermutohedralLatticeCPU.h:315-316).
void plref_matrix(void* h, int* vertex_out, float* weight_out) {
    get_matrix<float>(h, vertex_out, weight_out);
}
void plref_matrix_f64(void* h, int* vertex_out, double* weight_out) {
    get_matrix<double>(h, vertex_out, weight_out);
}

void plref_free(void* h) { free_run<float>(h); }
void plref_free_f64(void* h) { free_run<double>(h); }

// Timed CPU baseline.  reference may be NULL when n_ref_channels == 0.  min_vertices as in
// plref_filter.  Returns wall seconds (steady_clock), or -1 if a pre-sized table grew.
double plref_filter_batch(float* out, const float* in, const float* reference, int batch, int n,
                          int n_in_channels, int n_ref_channels, int n_sdims, const int* sdims,
                          float spatial_std, float feature_std, int reverse,
                          long long min_vertices, int threads) {
    return run_batch<float>(out, in, reference, batch, n, n_in_channels, n_ref_channels, n_sdims,
                            sdims, spatial_std, feature_std, reverse, min_vertices, threads);
}
double plref_filter_batch_f64(double* out, const double* in, const double* reference, int batch,
                              int n, int n_in_channels, int n_ref_channels, int n_sdims,
                              const int* sdims, double spatial_std, double feature_std, int reverse,
                              long long min_vertices, int threads) {
    return run_batch<double>(out, in, reference, batch, n, n_in_channels, n_ref_channels, n_sdims,
                             sdims, spatial_std, feature_std, reverse, min_vertices, threads);
}

}  // extern "C"
