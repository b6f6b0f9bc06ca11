// Per-point lattice geometry: elevate a pd-dimensional feature vector onto the hyperplane, find
// the enclosing simplex and the barycentric weights.  Every floating-point operation is done in
// the precision and order of the reference CPU implementation
// (src/PermutohedralLatticeCPU.h:220-286, T = float), because vertex keys must match it exactly:
// single roundings via __f*_rn (never contracted into FMAs).  Conversions and double arithmetic are
// avoided where an all-float, all-ALU formulation provably selects the same simplex (see
// find_simplex); the weights agree with the reference to the last bit except in the rare cases where
// its float(double(x) * (1/(pd+1))) double rounding differs from a correctly rounded product.
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
#define PL_FMA(a, b, c) __fmaf_rn((a), (b), (c))
#define PL_F2BITS(x) __float_as_int(x)
#define PL_BITS2F(x) __int_as_float(x)
#else
#include <cmath>
#define PL_FMUL(a, b) ((a) * (b))
#define PL_FADD(a, b) ((a) + (b))
#define PL_FSUB(a, b) ((a) - (b))
#define PL_FDIV(a, b) ((a) / (b))
#define PL_DMUL(a, b) ((a) * (b))
#define PL_DADD(a, b) ((a) + (b))
#define PL_FMA(a, b, c) fmaf((a), (b), (c))
#include <cstring>
static inline int pl_f2bits(float x) { int i; std::memcpy(&i, &x, 4); return i; }
static inline float pl_bits2f(int i) { float x; std::memcpy(&x, &i, 4); return x; }
#define PL_F2BITS(x) pl_f2bits(x)
#define PL_BITS2F(x) pl_bits2f(x)
#endif

namespace pl {

// 1.5 * 2^23: adding it to |x| < 2^22 leaves the nearest integer in the low mantissa bits.
#define PL_ROUND_MAGIC 12582912.0f

// Integer value of a float that holds an integer of magnitude below 2^22 (no conversion unit).
PL_HD int exact_int(float x) { return PL_F2BITS(PL_FADD(x, PL_ROUND_MAGIC)) - 0x4B400000; }

// (float)c for 0 <= c < 2^23 (no conversion unit).
PL_HD float small_int_to_float(int c) { return PL_FSUB(PL_BITS2F(0x4B000000 | c), 8388608.0f); }

// Correctly rounded a / b from the correctly rounded reciprocal rcp_b = RN(1 / b): q = RN(a rcp_b),
// exact remainder r = a - b q by fused multiply-add, result RN(q + r rcp_b).  For finite operands
// whose quotient and remainder stay in the normal range this equals the IEEE quotient.
PL_HD float div_by_rcp(float a, float b, float rcp_b) {
    const float q = PL_FMUL(a, rcp_b);
    const float r = PL_FMA(-b, q, a);
    return PL_FMA(r, rcp_b, q);
}

template <int PD>
struct Simplex {
    int rem0[PD + 1];  // nearest remainder-0 lattice point, per coordinate (multiple of PD+1)
    int rank[PD + 1];  // rank of each coordinate's residual, 0..PD
    float el[PD + 1];  // elevated position
    float rem0f[PD + 1];  // rem0 as float
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

    // Nearest remainder-0 point per coordinate.  The reference takes v = float(double(el) / (PD+1)),
    // up = ceil(v) (PD+1), down = floor(v) (PD+1) and picks up iff up - el < el - down.  Whenever v is
    // not within rounding of an integer, floor(el * (1/(PD+1))) in float is the same floor and
    // up = down + PD + 1; when it is, both candidate pairs contain the same winner with a margin of
    // a whole cell, so the choice below is identical in every case.  floor() by the add-magic trick.
    const float inv_f = 1.0f / (float)(PD + 1);
    int sum = 0;
#pragma unroll
    for (int i = 0; i <= PD; i++) {
        const float v = PL_FMUL(s.el[i], inv_f);
        float fl = PL_FSUB(PL_FADD(v, PL_ROUND_MAGIC), PL_ROUND_MAGIC);   // nearest integer
        fl = (fl > v) ? PL_FSUB(fl, 1.0f) : fl;                          // -> floor
        const float down = PL_FMUL(fl, (float)(PD + 1));                 // exact: small integers
        const float up = PL_FADD(down, (float)(PD + 1));
        s.rem0f[i] = (PL_FSUB(up, s.el[i]) < PL_FSUB(s.el[i], down)) ? up : down;
        s.rem0[i] = exact_int(s.rem0f[i]);
        sum += s.rem0[i];
    }
    sum /= (PD + 1);

    float d[PD + 1];
#pragma unroll
    for (int i = 0; i <= PD; i++) {
        d[i] = PL_FSUB(s.el[i], s.rem0f[i]);
        s.rank[i] = 0;
    }
#pragma unroll
    for (int i = 0; i < PD; i++) {
#pragma unroll
        for (int j = i + 1; j <= PD; j++) {
            const int lt = d[i] < d[j] ? 1 : 0;   // arithmetic on the predicate: no branches
            s.rank[i] += lt;
            s.rank[j] += 1 - lt;
        }
    }
#pragma unroll
    for (int i = 0; i <= PD; i++) {
        s.rank[i] += sum;
        // wrap into 0..PD: +1 cell when below, -1 cell when above (selects, no branches)
        const int wrap = (s.rank[i] < 0 ? 1 : 0) - (s.rank[i] > PD ? 1 : 0);
        s.rank[i] += wrap * (PD + 1);
        s.rem0[i] += wrap * (PD + 1);
        s.rem0f[i] = (wrap > 0)   ? PL_FADD(s.rem0f[i], (float)(PD + 1))
                     : (wrap < 0) ? PL_FSUB(s.rem0f[i], (float)(PD + 1))
                                  : s.rem0f[i];
    }
}

// Barycentric weights, one per remainder (src/PermutohedralLatticeCPU.h:275-286).  The reference
// scatters +delta_i to slot pd-rank_i and -delta_i to slot pd-rank_i+1 of a zeroed array; each
// slot k in 1..pd thus ends as fl(delta[rank = pd-k] - delta[rank = pd-k+1]) whatever the order,
// slot pd+1 as -delta[rank = 0], and slot 0 gets the wrap-around in double.  Written here without
// data-dependent array indexing.
template <int PD>
PL_HD void barycentric(const Simplex<PD>& s, float* bary /* PD+1 */) {
    // delta_i = (el_i - rem0_i) / (PD+1): the reference multiplies by the double 1/(PD+1) and rounds
    // to float; here the same product is formed in float-float arithmetic (c = ch + cl), which gives
    // the correctly rounded float without conversions.
    const double c = 1.0 / (PD + 1);
    const float ch = (float)c;
    const float cl = (float)(c - (double)ch);
    float by_rank[PD + 1];
#pragma unroll
    for (int q = 0; q <= PD; q++) by_rank[q] = 0.f;
#pragma unroll
    for (int i = 0; i <= PD; i++) {
        const float d = PL_FSUB(s.el[i], s.rem0f[i]);
        const float p = PL_FMUL(d, ch);
        const float e = PL_FMA(d, ch, -p);             // exact error of p
        const float delta = PL_FADD(p, PL_FMA(d, cl, e));
#pragma unroll
        for (int q = 0; q <= PD; q++) by_rank[q] = (s.rank[i] == q) ? delta : by_rank[q];   // select, not branch
    }
#pragma unroll
    for (int k = 1; k <= PD; k++) bary[k] = PL_FSUB(by_rank[PD - k], by_rank[PD - k + 1]);
    bary[0] = (float)PL_DADD((double)by_rank[PD], PL_DADD(1.0, (double)(-by_rank[0])));
}

// Coordinate i (< PD) of the remainder-r vertex of the simplex (src/PermutohedralLatticeCPU.h:297-304).
template <int PD>
PL_HD int16_t vertex_coord(const Simplex<PD>& s, int i, int r) {
    const int k = s.rem0[i] + r - ((s.rank[i] > PD - r) ? PD + 1 : 0);
    return (int16_t)k;
}

// ---------------------------------------------------------------------------------------------
// T = double (src/PermutohedralLatticeCPU.h:220-286 with T = double).  Written exactly as the
// reference computes it: there is nothing to gain from avoiding conversions here.  One quirk is
// kept: the elevation step holds position * scale in a float (:226), and multiplies it by the
// loop index in float, whatever T is.
// ---------------------------------------------------------------------------------------------
template <int PD>
struct Simplex64 {
    int rem0[PD + 1];
    int rank[PD + 1];
    double el[PD + 1];
};

template <int PD>
PL_HD void find_simplex_f64(const double* pos, const double* scale, Simplex64<PD>& s) {
    double sm = 0.0;
#pragma unroll
    for (int i = PD; i > 0; i--) {
        const float cf = (float)PL_DMUL(pos[i - 1], scale[i - 1]);
        s.el[i] = PL_DADD(sm, -(double)PL_FMUL((float)i, cf));
        sm = PL_DADD(sm, (double)cf);
    }
    s.el[0] = sm;
    const double inv = 1.0 / (PD + 1);
    int sum = 0;
#pragma unroll
    for (int i = 0; i <= PD; i++) {
        const double v = PL_DMUL(s.el[i], inv);
        const double up = PL_DMUL(ceil(v), (double)(PD + 1));
        const double down = PL_DMUL(floor(v), (double)(PD + 1));
        const double r0 = (PL_DADD(up, -s.el[i]) < PL_DADD(s.el[i], -down)) ? up : down;
        s.rem0[i] = (int)(int16_t)r0;
        sum += s.rem0[i];
    }
    sum /= (PD + 1);
    double d[PD + 1];
#pragma unroll
    for (int i = 0; i <= PD; i++) {
        d[i] = PL_DADD(s.el[i], -(double)s.rem0[i]);
        s.rank[i] = 0;
    }
#pragma unroll
    for (int i = 0; i < PD; i++) {
#pragma unroll
        for (int j = i + 1; j <= PD; j++) {
            const int lt = d[i] < d[j] ? 1 : 0;
            s.rank[i] += lt;
            s.rank[j] += 1 - lt;
        }
    }
#pragma unroll
    for (int i = 0; i <= PD; i++) {
        s.rank[i] += sum;
        const int wrap = (s.rank[i] < 0 ? 1 : 0) - (s.rank[i] > PD ? 1 : 0);
        s.rank[i] += wrap * (PD + 1);
        s.rem0[i] += wrap * (PD + 1);
    }
}

template <int PD>
PL_HD void barycentric_f64(const Simplex64<PD>& s, double* bary /* PD+1 */) {
    const double inv = 1.0 / (PD + 1);
    double by_rank[PD + 1];
#pragma unroll
    for (int q = 0; q <= PD; q++) by_rank[q] = 0.0;
#pragma unroll
    for (int i = 0; i <= PD; i++) {
        const double delta = PL_DMUL(PL_DADD(s.el[i], -(double)s.rem0[i]), inv);
#pragma unroll
        for (int q = 0; q <= PD; q++) by_rank[q] = (s.rank[i] == q) ? delta : by_rank[q];
    }
#pragma unroll
    for (int k = 1; k <= PD; k++) bary[k] = PL_DADD(by_rank[PD - k], -by_rank[PD - k + 1]);
    bary[0] = PL_DADD(by_rank[PD], PL_DADD(1.0, -by_rank[0]));
}

template <int PD>
PL_HD int16_t vertex_coord(const Simplex64<PD>& s, int i, int r) {
    const int k = s.rem0[i] + r - ((s.rank[i] > PD - r) ? PD + 1 : 0);
    return (int16_t)k;
}

}  // namespace pl
