// Per-point lattice geometry: elevate a pd-dimensional feature vector onto the hyperplane, find
// the enclosing simplex and the barycentric weights.  Every floating-point operation is done in
// the precision and order of the reference CPU implementation
// (src/PermutohedralLatticeCPU.h:220-286, T = float), because vertex keys must match it exactly:
// single roundings via __f*_rn (never contracted into FMAs), the multiply by 1/(pd+1) in double.
//
// Compiles for the host too (PL_HD), so the arithmetic can be checked without a GPU.
#pragma once
#include <stdint.h>

#ifdef __CUDACC__
#define PL_HD __host__ __device__ __forceinline__
#else
#define PL_HD inline
#endif

#ifdef __CUDA_ARCH__
#define PL_FMUL(a, b) __fmul_rn((a), (b))
#define PL_FADD(a, b) __fadd_rn((a), (b))
#define PL_FSUB(a, b) __fsub_rn((a), (b))
#define PL_FDIV(a, b) __fdiv_rn((a), (b))
#define PL_DMUL(a, b) __dmul_rn((a), (b))
#define PL_DADD(a, b) __dadd_rn((a), (b))
#else
#include <cmath>
#define PL_FMUL(a, b) ((a) * (b))
#define PL_FADD(a, b) ((a) + (b))
#define PL_FSUB(a, b) ((a) - (b))
#define PL_FDIV(a, b) ((a) / (b))
#define PL_DMUL(a, b) ((a) * (b))
#define PL_DADD(a, b) ((a) + (b))
#endif

namespace pl {

template <int PD>
struct Simplex {
    int rem0[PD + 1];  // nearest remainder-0 lattice point, per coordinate (multiple of PD+1)
    int rank[PD + 1];  // rank of each coordinate's residual, 0..PD
    float el[PD + 1];  // elevated position
};

// src/PermutohedralLatticeCPU.h:220-273 (embed_position_vector, find_enclosing_simplex).
// scale[i] must be the host-computed factors of compute_scale_factor (:194-217).
template <int PD>
PL_HD void find_simplex(const float* pos, const float* scale, Simplex<PD>& s) {
    float sm = 0.f;
#pragma unroll
    for (int i = PD; i > 0; i--) {
        float cf = PL_FMUL(pos[i - 1], scale[i - 1]);
        s.el[i] = PL_FSUB(sm, PL_FMUL((float)i, cf));
        sm = PL_FADD(sm, cf);
    }
    s.el[0] = sm;

    const double inv = 1.0 / (PD + 1);
    float rem0f[PD + 1];
    int sum = 0;
#pragma unroll
    for (int i = 0; i <= PD; i++) {
        float v = (float)PL_DMUL((double)s.el[i], inv);
        float up = ceilf(v) * (float)(PD + 1);    // exact: small integers
        float down = floorf(v) * (float)(PD + 1);
        rem0f[i] = (PL_FSUB(up, s.el[i]) < PL_FSUB(s.el[i], down)) ? up : down;
        s.rem0[i] = (int)rem0f[i];
        sum += s.rem0[i];
    }
    sum /= (PD + 1);

    float d[PD + 1];
#pragma unroll
    for (int i = 0; i <= PD; i++) {
        d[i] = PL_FSUB(s.el[i], rem0f[i]);
        s.rank[i] = 0;
    }
#pragma unroll
    for (int i = 0; i < PD; i++) {
#pragma unroll
        for (int j = i + 1; j <= PD; j++) {
            if (d[i] < d[j])
                s.rank[i]++;
            else
                s.rank[j]++;
        }
    }
#pragma unroll
    for (int i = 0; i <= PD; i++) {
        s.rank[i] += sum;
        if (s.rank[i] < 0) {
            s.rank[i] += PD + 1;
            s.rem0[i] += PD + 1;
        } else if (s.rank[i] > PD) {
            s.rank[i] -= PD + 1;
            s.rem0[i] -= PD + 1;
        }
    }
}

// Barycentric weights, one per remainder (src/PermutohedralLatticeCPU.h:275-286).  The reference
// scatters +delta_i to slot pd-rank_i and -delta_i to slot pd-rank_i+1 of a zeroed array; each
// slot k in 1..pd thus ends as fl(delta[rank = pd-k] - delta[rank = pd-k+1]) whatever the order,
// slot pd+1 as -delta[rank = 0], and slot 0 gets the wrap-around in double.  Written here without
// data-dependent array indexing.
template <int PD>
PL_HD void barycentric(const Simplex<PD>& s, float* bary /* PD+1 */) {
    const double inv = 1.0 / (PD + 1);
    float by_rank[PD + 1];
#pragma unroll
    for (int q = 0; q <= PD; q++) by_rank[q] = 0.f;
#pragma unroll
    for (int i = 0; i <= PD; i++) {
        float delta = (float)PL_DMUL((double)PL_FSUB(s.el[i], (float)s.rem0[i]), inv);
#pragma unroll
        for (int q = 0; q <= PD; q++)
            if (s.rank[i] == q) by_rank[q] = delta;
    }
#pragma unroll
    for (int k = 1; k <= PD; k++) bary[k] = PL_FSUB(by_rank[PD - k], by_rank[PD - k + 1]);
    bary[0] = (float)PL_DADD((double)by_rank[PD], PL_DADD(1.0, (double)(-by_rank[0])));
}

// Coordinate i (< PD) of the remainder-r vertex of the simplex (src/PermutohedralLatticeCPU.h:297-304).
template <int PD>
PL_HD int16_t vertex_coord(const Simplex<PD>& s, int i, int r) {
    int k = s.rem0[i] + r;
    if (s.rank[i] > PD - r) k -= PD + 1;
    return (int16_t)k;
}

}  // namespace pl
