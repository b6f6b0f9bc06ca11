// Host-side build of the product's per-point lattice geometry (csrc/simplex.cuh), so its key and
// weight arithmetic can be compared with the CPU oracle without a GPU.
#include "simplex.cuh"

template <int PD>
static void run(const float* pos, const float* scale, int n, int16_t* keys, float* weights) {
    for (int p = 0; p < n; p++) {
        pl::Simplex<PD> s;
        pl::find_simplex<PD>(pos + (size_t)p * PD, scale, s);
        float b[PD + 1];
        pl::barycentric<PD>(s, b);
        for (int r = 0; r <= PD; r++) {
            weights[(size_t)p * (PD + 1) + r] = b[r];
            for (int i = 0; i < PD; i++)
                keys[((size_t)p * (PD + 1) + r) * PD + i] = pl::vertex_coord<PD>(s, i, r);
        }
    }
}

extern "C" int simplex_host(const float* pos, const float* scale, int n, int pd, int16_t* keys,
                            float* weights) {
    switch (pd) {
        case 2: run<2>(pos, scale, n, keys, weights); return 0;
        case 3: run<3>(pos, scale, n, keys, weights); return 0;
        case 4: run<4>(pos, scale, n, keys, weights); return 0;
        case 5: run<5>(pos, scale, n, keys, weights); return 0;
        case 16: run<16>(pos, scale, n, keys, weights); return 0;
    }
    return 1;
}

template <int PD>
static void run64(const double* pos, const double* scale, int n, int16_t* keys, double* weights) {
    for (int p = 0; p < n; p++) {
        pl::Simplex64<PD> s;
        pl::find_simplex_f64<PD>(pos + (size_t)p * PD, scale, s);
        double b[PD + 1];
        pl::barycentric_f64<PD>(s, b);
        for (int r = 0; r <= PD; r++) {
            weights[(size_t)p * (PD + 1) + r] = b[r];
            for (int i = 0; i < PD; i++)
                keys[((size_t)p * (PD + 1) + r) * PD + i] = pl::vertex_coord<PD>(s, i, r);
        }
    }
}

extern "C" int simplex_host_f64(const double* pos, const double* scale, int n, int pd, int16_t* keys,
                                double* weights) {
    switch (pd) {
        case 2: run64<2>(pos, scale, n, keys, weights); return 0;
        case 3: run64<3>(pos, scale, n, keys, weights); return 0;
        case 4: run64<4>(pos, scale, n, keys, weights); return 0;
        case 5: run64<5>(pos, scale, n, keys, weights); return 0;
        case 16: run64<16>(pos, scale, n, keys, weights); return 0;
    }
    return 1;
}

// a / b through the reciprocal-based division used for the features; rcp = RN(1 / b).
extern "C" void div_by_rcp_host(const float* a, float b, int n, float* out) {
    const float rcp = 1.0f / b;
    for (int i = 0; i < n; i++) out[i] = pl::div_by_rcp(a[i], b, rcp);
}
extern "C" float small_int_to_float_host(int c) { return pl::small_int_to_float(c); }
