// Host-side build of the dense index of spatial-only calls (csrc/direct_bounds.h), so that its bounds
// can be checked against the CPU oracle's vertex keys without a GPU.
#include "direct_bounds.h"

// Returns 1 and fills lo0, dlo[8], ext[8], cells when the index can be used, else 0.
extern "C" int direct_bounds_host(int pd, const int* sdims, float spatial_std, const float* scale, int batch,
                                  unsigned long long max_slots, int* lo0, int* dlo, unsigned* ext,
                                  unsigned long long* cells) {
    pl::Direct d;
    if (!pl::direct_bounds(d, pd, sdims, spatial_std, scale, batch, max_slots)) return 0;
    *lo0 = d.lo0;
    for (int i = 0; i < pl::DIRECT_MAX_DIMS; i++) {
        dlo[i] = d.dlo[i];
        ext[i] = d.ext[i];
    }
    *cells = d.cells;
    return 1;
}

// slots[n] <- slot of each key (n rows of pd int16 coordinates, batch item 0); returns how many keys
// fall outside the index.
extern "C" int direct_slots_host(int pd, const int* sdims, float spatial_std, const float* scale,
                                 const short* keys, int n, unsigned long long* slots) {
    pl::Direct d;
    if (!pl::direct_bounds(d, pd, sdims, spatial_std, scale, 1, ~0ull >> 1)) return -1;
    int outside = 0;
    for (int i = 0; i < n; i++)
        if (!pl::direct_slot_host(d, pd, keys + (size_t)i * pd, 0, slots[i])) outside++;
    return outside;
}
