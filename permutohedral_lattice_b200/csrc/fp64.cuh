// T = double: splat, blur and slice over rows of doubles.  The lattice structure (keys, table,
// vertex and neighbour tables) comes from the same kernels as for float; only the geometry
// arithmetic and the value rows differ.  These kernels favour plainness over the last bit of speed:
// a warp walks sorted splats (or points) with its lanes spread over the channels.
#pragma once
#include "common.cuh"
#include "splat.cuh"

namespace pl {

// Doubles of a vertex row: vd padded to a multiple of 2 (16-byte rows).
__host__ __device__ __forceinline__ int padded_vd_f64(int vd) { return (vd + 1) & ~1; }

template <int PD>
struct Splat64 {
    static constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS;
    static constexpr size_t BYTES = sizeof(double) * SPLATS + sizeof(uint2) * SPLATS + sizeof(int) * SPLATS +
                                    sizeof(int) * TP;
};

// V[vertex] += sum over the tile's splats of weight * [input channels, 1]
// (src/PermutohedralLatticeCPU.h:306-313).  The tile's splats are counting-sorted by entry; every warp
// walks a contiguous chunk of the sorted list, lanes over channels, sums each entry's run in a
// register and adds it to the vertex row with one reduction per channel.
template <int PD>
__global__ void __launch_bounds__(Cfg<PD>::TP)
splat_tiles_f64(Geom g, const double* __restrict__ input, Header* hdr, const int2* __restrict__ tile_info,
                const u16* __restrict__ rec, const double* __restrict__ rec_w,
                const u32* __restrict__ list_ref, double* __restrict__ v0, int vd) {
    constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS, NW = TP / 32;
    const int C = vd - 1, VP = padded_vd_f64(vd);
    extern __shared__ __align__(16) unsigned char smem_raw[];
    double* w_s = reinterpret_cast<double*>(smem_raw);            // [SPLATS] weight of splat r * TP + point
    uint2* sorted_s = reinterpret_cast<uint2*>(w_s + SPLATS);     // [SPLATS] (point | entry << 16, remainder)
    int* cur_s = reinterpret_cast<int*>(sorted_s + SPLATS);       // [SPLATS]
    int* prow_s = cur_s + SPLATS;                                 // [TP]
    __shared__ int wsum_s[32];
    if (call_failed(hdr)) return;
    const TilePos tpos = this_tile(g);
    const int tid = threadIdx.x, tile = tpos.tile, lane = tid & 31, warp = tid >> 5;
    const int2 info = tile_info[tile];
    const int base = info.x, nloc = info.y;
    int item, pix;
    const bool valid = tile_point(g, tpos, tid, item, pix);
    prow_s[tid] = valid ? item * g.n + pix : -1;
    for (int i = tid; i < nloc; i += TP) cur_s[i] = 0;
    const int nvalid = __syncthreads_count(valid);
    int l[PD + 1];
    float tag[PD + 1];   // the sorted list carries the remainder in place of a float weight
    const u16* rec_tile = rec + (size_t)tile * SPLATS;
    const double* recw_tile = rec_w + (size_t)tile * SPLATS;
#pragma unroll
    for (int r = 0; r <= PD; r++) {
        l[r] = valid ? rec_tile[r * TP + tid] : 0;
        w_s[r * TP + tid] = valid ? recw_tile[r * TP + tid] : 0.0;
        tag[r] = __int_as_float(r);
    }
    SplatCommon<PD>::template sort_splats<0>(valid, l, tag, nloc, sorted_s, cur_s, nullptr, wsum_s);

    const int total = nvalid * (PD + 1);
    const int chunk = (total + NW - 1) / NW;
    const int beg = warp * chunk, end = min(total, beg + chunk);
    if (beg >= end) return;
    for (int j0 = 0; j0 < vd; j0 += 32) {
        const int j = j0 + lane;
        double acc = 0.0;
        int cur = (int)(sorted_s[beg].x >> 16);
        for (int sidx = beg; sidx < end; sidx++) {
            const uint2 pw = sorted_s[sidx];
            const int e = (int)(pw.x >> 16);
            if (e != cur) {
                if (j < vd) red_add_f64(v0 + (size_t)list_ref[base + cur] * VP + j, acc);
                acc = 0.0;
                cur = e;
            }
            if (j < vd) {
                const int p = (int)(pw.x & 0xFFFFu);
                const double wt = w_s[(int)pw.y * TP + p];
                acc = PL_DADD(acc, (j < C) ? PL_DMUL(wt, __ldg(input + (size_t)prow_s[p] * C + j)) : wt);
            }
        }
        if (j < vd) red_add_f64(v0 + (size_t)list_ref[base + cur] * VP + j, acc);
    }
}

// One [1 2 1]/4 pass along a lattice axis (src/PermutohedralLatticeCPU.h:403-405).  One double2 per thread.
__global__ void __launch_bounds__(256)
blur_axis_f64(const Header* hdr, const int* __restrict__ nbr_axis, const double* __restrict__ src,
              double* __restrict__ dst, int ppr /* double2 per row */) {
    if (hdr->status != 0) return;
    const u32 M = hdr->num_vertices;
    const u64 items = (u64)M * ppr;
    const double2* __restrict__ s = reinterpret_cast<const double2*>(src);
    double2* __restrict__ d = reinterpret_cast<double2*>(dst);
    const int2* __restrict__ nb = reinterpret_cast<const int2*>(nbr_axis);
    const double2 zero = make_double2(0.0, 0.0);
    for (u64 e = (u64)blockIdx.x * blockDim.x + threadIdx.x; e < items; e += (u64)gridDim.x * blockDim.x) {
        const u32 v = (u32)(e / ppr);
        const int j = (int)(e - (u64)v * ppr);
        const int2 n = __ldg(nb + v);
        const double2 b = s[e];
        const double2 a = (n.x >= 0) ? s[(u64)n.x * ppr + j] : zero;
        const double2 c = (n.y >= 0) ? s[(u64)n.y * ppr + j] : zero;
        d[e] = make_double2(PL_DADD(PL_DADD(PL_DMUL(0.25, a.x), PL_DMUL(0.5, b.x)), PL_DMUL(0.25, c.x)),
                            PL_DADD(PL_DADD(PL_DMUL(0.25, a.y), PL_DMUL(0.5, b.y)), PL_DMUL(0.25, c.y)));
    }
}

// Slice (src/PermutohedralLatticeCPU.h:333-352): per point and channel the weighted sum over the
// remainders in ascending order, then one multiply by the reciprocal of the homogeneous channel.
// A warp takes 32 points of the tile, one after the other, lanes over channels.
template <int PD>
__global__ void __launch_bounds__(Cfg<PD>::TP)
slice_tiles_f64(Geom g, double* __restrict__ output, const Header* hdr, const int2* __restrict__ tile_info,
                const u16* __restrict__ rec, const double* __restrict__ rec_w,
                const u32* __restrict__ list_ref, const double* __restrict__ vsrc, int vd) {
    constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS;
    const int C = vd - 1, VP = padded_vd_f64(vd);
    __shared__ double w_s[SPLATS];
    __shared__ u32 v_s[SPLATS];
    __shared__ int prow_s[TP];
    if (call_failed(hdr)) {
        poison_tile_output(g, output, C);
        return;
    }
    const TilePos tpos = this_tile(g);
    const int tid = threadIdx.x, tile = tpos.tile, lane = tid & 31, warp = tid >> 5;
    const int base = tile_info[tile].x;
    int item, pix;
    const bool valid = tile_point(g, tpos, tid, item, pix);
    prow_s[tid] = valid ? item * g.n + pix : -1;
    const u16* rec_tile = rec + (size_t)tile * SPLATS;
    const double* recw_tile = rec_w + (size_t)tile * SPLATS;
#pragma unroll
    for (int r = 0; r <= PD; r++) {
        w_s[r * TP + tid] = valid ? recw_tile[r * TP + tid] : 0.0;
        v_s[r * TP + tid] = valid ? list_ref[base + rec_tile[r * TP + tid]] : 0u;
    }
    __syncthreads();
    for (int i = 0; i < 32; i++) {
        const int p = warp * 32 + i;
        const int row = prow_s[p];
        if (row < 0) continue;
        double norm = 0.0;
#pragma unroll
        for (int r = 0; r <= PD; r++)
            norm = PL_DADD(norm, PL_DMUL(w_s[r * TP + p], __ldg(vsrc + (size_t)v_s[r * TP + p] * VP + C)));
        const double inv = __ddiv_rn(1.0, norm);
        for (int j = lane; j < C; j += 32) {
            double acc = 0.0;
#pragma unroll
            for (int r = 0; r <= PD; r++)
                acc = PL_DADD(acc, PL_DMUL(w_s[r * TP + p], __ldg(vsrc + (size_t)v_s[r * TP + p] * VP + j)));
            output[(size_t)row * C + j] = PL_DMUL(acc, inv);
        }
    }
}

}  // namespace pl
