// Stand-alone positions kernel and the read-out of the lattice structure for verification.
#pragma once
#include "common.cuh"

namespace pl {

// ---------------------------------------------------------------------------------------------
// positions kernel (the standalone ComputeKernel functor) and lattice export
// ---------------------------------------------------------------------------------------------
__global__ void positions_kernel_f64(const double* __restrict__ reference, double* __restrict__ positions,
                                     int n, int R, int n_sdims, Geom g) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const int pd = n_sdims + R;
    int divisor = 1;
    for (int s = n_sdims - 1; s >= 0; s--) {
        positions[(size_t)pd * idx + s] = __ddiv_rn((double)((idx / divisor) % g.sdims[s]), g.spatial_std_d);
        divisor *= g.sdims[s];
    }
    for (int c = 0; c < R; c++)
        positions[(size_t)pd * idx + n_sdims + c] = __ddiv_rn(reference[(size_t)idx * R + c], g.feature_std_d);
}

__global__ void positions_kernel(const float* __restrict__ reference, float* __restrict__ positions,
                                 int n, int R, int n_sdims, Geom g) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const int pd = n_sdims + R;
    int divisor = 1;
    for (int s = n_sdims - 1; s >= 0; s--) {
        positions[(size_t)pd * idx + s] = PL_FDIV((float)((idx / divisor) % g.sdims[s]), g.spatial_std);
        divisor *= g.sdims[s];
    }
    for (int c = 0; c < R; c++)
        positions[(size_t)pd * idx + n_sdims + c] = PL_FDIV(reference[(size_t)idx * R + c], g.feature_std);
}

template <int PD, typename R = float>
__global__ void __launch_bounds__(Cfg<PD>::TP)
export_points(Geom g, const Header* hdr, const int2* __restrict__ tile_info, const u16* __restrict__ rec,
              const R* __restrict__ rec_w, const u32* __restrict__ list_ref,
              int32_t* __restrict__ pixel_vertex, R* __restrict__ pixel_weight) {
    constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS;
    if (hdr->status != 0) return;
    const TilePos tpos = this_tile(g);
    const int tid = threadIdx.x, tile = tpos.tile;
    int item, pix;
    if (!tile_point(g, tpos, tid, item, pix)) return;
    const int base = tile_info[tile].x;
    const u16* rec_tile = rec + (size_t)tile * SPLATS;
    const R* recw_tile = rec_w + (size_t)tile * SPLATS;
    const size_t o = ((size_t)item * g.n + pix) * (PD + 1);
#pragma unroll
    for (int r = 0; r <= PD; r++) {
        if (pixel_vertex) pixel_vertex[o + r] = (int32_t)list_ref[base + rec_tile[r * TP + tid]];
        if (pixel_weight) pixel_weight[o + r] = recw_tile[r * TP + tid];
    }
}

template <int PD>
__global__ void export_vertices(const Header* hdr, const Key<Cfg<PD>::KW>* __restrict__ vkeys, long long max_vertices,
                                int16_t* __restrict__ vertex_keys, int32_t* __restrict__ vertex_item) {
    constexpr int KW = Cfg<PD>::KW;
    if (hdr->status != 0) return;
    const u32 M = hdr->num_vertices;
    for (u64 v = (u64)blockIdx.x * blockDim.x + threadIdx.x; v < M && v < (u64)max_vertices;
         v += (u64)gridDim.x * blockDim.x) {
        const Key<KW> k = vkeys[v];
        if (vertex_keys) {
#pragma unroll
            for (int i = 0; i < PD; i++) vertex_keys[v * PD + i] = (int16_t)(key_get<KW>(k, i) ^ 0x8000);
        }
        if (vertex_item) vertex_item[v] = (int32_t)key_get<KW>(k, PD);
    }
}

}  // namespace pl
