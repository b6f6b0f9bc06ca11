// Host-side arithmetic of the direct index of spatial-only calls (plain C++, no CUDA: the CPU tests
// compile this file on its own).  See direct_index.cuh for the kernels that use the result.
#pragma once
#include <cmath>
#include <cstring>

namespace pl {

constexpr int DIRECT_MAX_DIMS = 8;

// A lattice point has all its coordinates congruent modulo pd+1, so with k_0 the first stored
// coordinate, (k_i - k_0) / (pd+1) is an integer.  The dense index of a key is
//   (((k_0 - lo0) * ext[1] + (k_1 - k_0)/(pd+1) - dlo[1]) * ext[2] + ...) + item * cells.
struct Direct {
    int on;
    int lo0;                         // smallest first coordinate
    int dlo[DIRECT_MAX_DIMS];        // i >= 1: smallest (k_i - k_0) / (pd+1)
    unsigned ext[DIRECT_MAX_DIMS];   // extent of each index coordinate
    unsigned long long cells;        // slots per batch item
    unsigned long long slots;        // batch * cells
};

// Bounds of the vertex keys that a grid of sdims[0..pd-1] points can create when feature j of a point
// is c_j / spatial_std (0 <= c_j < sdims[j]), and the dense index built on them.  The elevated
// coordinates (src/PermutohedralLatticeCPU.h:220-231) are el_0 = sum_j cf_j and
// el_i = sum_{j>=i} cf_j - i cf_{i-1} with cf_j = feature_j * scale_j >= 0, so each lies in an interval
// known from the grid's size.  A vertex of the enclosing simplex is within 2.5 (pd+1) of the point in
// every coordinate (nearest multiple of pd+1, one wrap of pd+1, remainder offsets up to pd); the margin
// is wider than that and also covers the rounding of the float arithmetic.
// Returns false (d.on = 0) when the index cannot be used: bad arguments, coordinates beyond 16 bits,
// or more than max_slots slots for `batch` items.
inline bool direct_bounds(Direct& d, int pd, const int* sdims, float spatial_std, const float* scale, int batch,
                          unsigned long long max_slots) {
    std::memset(&d, 0, sizeof(d));
    if (pd < 1 || pd > DIRECT_MAX_DIMS || batch < 1) return false;
    if (!(spatial_std > 0.f) || !std::isfinite(spatial_std)) return false;
    double cf[DIRECT_MAX_DIMS];
    double sum_all = 0;
    for (int j = 0; j < pd; j++) {
        if (sdims[j] < 1) return false;
        cf[j] = (double)(sdims[j] - 1) / (double)spatial_std * (double)scale[j];
        if (!(cf[j] < 30000.0)) return false;
        sum_all += cf[j];
    }
    const double margin = 3.0 * (pd + 1) + 2.0;
    if (sum_all + margin > 30000.0) return false;   // coordinates are 16-bit, as in the reference
    d.lo0 = (int)std::floor(-margin);
    d.ext[0] = (unsigned)((int)std::ceil(sum_all + margin) - d.lo0 + 1);
    unsigned long long cells = d.ext[0];
    for (int i = 1; i < pd; i++) {
        // k_i - k_0 follows el_i - el_0 = -(i cf_{i-1} + sum_{j<i} cf_j)
        double span = i * cf[i - 1];
        for (int j = 0; j < i; j++) span += cf[j];
        const int lo = (int)std::floor((-span - 2 * margin) / (pd + 1));
        const int hi = (int)std::ceil((2 * margin) / (pd + 1));
        d.dlo[i] = lo;
        d.ext[i] = (unsigned)(hi - lo + 1);
        cells *= d.ext[i];
        if (cells > (1ull << 32)) return false;
    }
    d.cells = cells;
    d.slots = cells * (unsigned long long)batch;
    if (d.slots > max_slots || d.slots >= 0xFFFFFFFFull) return false;   // entry numbers must fit a 32-bit slot
    d.on = 1;
    return true;
}

// Slot of the key with stored coordinates k[0..pd-1] of batch item `item`; false when outside the index.
inline bool direct_slot_host(const Direct& d, int pd, const short* k, int item, unsigned long long& slot) {
    const int k0 = k[0];
    const unsigned c0 = (unsigned)(k0 - d.lo0);
    bool ok = c0 < d.ext[0];
    unsigned long long idx = c0;
    for (int i = 1; i < pd; i++) {
        const int di = ((int)k[i] - k0) / (pd + 1);
        const unsigned ci = (unsigned)(di - d.dlo[i]);
        ok = ok && ci < d.ext[i];
        idx = idx * d.ext[i] + ci;
    }
    slot = (unsigned long long)item * d.cells + idx;
    return ok;
}

}  // namespace pl
