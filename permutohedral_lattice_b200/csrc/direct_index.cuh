// Direct indexing of lattice vertices for spatial-only filters (bilateral == 0: the features are the
// grid coordinates divided by one standard deviation; src/LatticeFilterKernel.cpp:137-142,
// Tests/PermutohedralLatticeGPU.cu:33-42).  The vertices such a call can touch lie in a bounded region
// of the lattice that the host knows before anything runs, so a vertex key maps to its own slot of a
// dense array: no hashing, no probing, no key comparison.  The kernels below stand in for clear_table,
// insert_entries and link_neighbours; everything before and after them is unchanged.
#pragma once
#include "common.cuh"
#include "direct_bounds.h"

namespace pl {

static_assert(DIRECT_MAX_DIMS == MAX_SDIMS, "the index has one coordinate per spatial dimension");

constexpr u32 DIRECT_EMPTY = 0xFFFFFFFFu;

// Slot of key k; false when k lies outside the indexed region (then no point can have created it).
template <int PD>
__device__ __forceinline__ bool direct_slot(const Direct& d, const Key<Cfg<PD>::KW>& k, u64& slot) {
    constexpr int KW = Cfg<PD>::KW;
    const int k0 = (int)key_get<KW>(k, 0) - 0x8000;
    const u32 c0 = (u32)(k0 - d.lo0);
    bool ok = c0 < d.ext[0];
    u64 idx = c0;
#pragma unroll
    for (int i = 1; i < PD; i++) {
        const int ki = (int)key_get<KW>(k, i) - 0x8000;
        const int di = (ki - k0) / (PD + 1);
        const u32 ci = (u32)(di - d.dlo[i]);
        ok = ok && ci < d.ext[i];
        idx = idx * d.ext[i] + ci;
    }
    slot = (u64)key_get<KW>(k, PD) * d.cells + idx;
    return ok;
}

__global__ void clear_direct(Header* hdr, u32* __restrict__ table, u64 slots) {
    after_previous_kernel();
    if (hdr->status != 0) return;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        u32 lg = 0;
        while ((1ull << lg) < slots) lg++;
        hdr->table_log2 = lg;
        hdr->direct = 1;
    }
    for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i < slots; i += (u64)gridDim.x * blockDim.x)
        table[i] = DIRECT_EMPTY;
}

// One 32-bit compare-and-swap per entry: the first entry to reach a slot owns a new vertex.
template <int PD>
__global__ void __launch_bounds__(256)
insert_direct(Header* hdr, Direct d, u32* __restrict__ table, const Key<Cfg<PD>::KW>* __restrict__ list_keys,
              u32* __restrict__ list_ref, u32* __restrict__ vid, Key<Cfg<PD>::KW>* __restrict__ vkeys,
              VertexInit vi) {
    after_previous_kernel();
    constexpr int KW = Cfg<PD>::KW;
    __shared__ InsertRound rd;
    if (threadIdx.x == 0) rd.count = 0;
    if (call_failed(hdr)) return;   // (its barrier also publishes rd.count)
    const u32 T = hdr->num_entries;
    const u32 stride = gridDim.x * 256u;
    for (u32 start = blockIdx.x * 256u; start < T;) {
        for (int c = 0; c < INSERT_CHUNKS && start < T; c++, start += stride) {
            const u32 t = start + threadIdx.x;
            bool winner = false;
            u64 s = 0;
            if (t < T) {
                u32 ref = t;
                if (direct_slot<PD>(d, list_keys[t], s)) {
                    const u32 cur = atomicCAS(&table[s], DIRECT_EMPTY, t);
                    winner = cur == DIRECT_EMPTY;
                    if (!winner) ref = cur;   // owning entry, or (VERTEX_FLAG set) the vertex itself
                } else {
                    atomicOr(&hdr->status, 1u << PL_INTERNAL_ERROR);   // the host's bounds missed a point's vertex
                }
                list_ref[t] = ref;
            }
            round_add_winner(rd, winner, t, (u32)s);
        }
        finish_round<KW>(hdr, rd, list_keys, vid, vkeys, vi,
                         [&](u32 slot, u32 v) { table[slot] = VERTEX_FLAG | v; });
    }
}

// The "+" neighbour of vertex v along axis a (src/PermutohedralLatticeCPU.h:381-388) by one load of
// its slot (every slot carries a vertex index by now); the same result fills that neighbour's "-" slot.
template <int PD>
__global__ void __launch_bounds__(256)
link_neighbours_direct(const Header* hdr, Direct d, const u32* __restrict__ table, u32* __restrict__ list_ref,
                       const u32* __restrict__ vid, const Key<Cfg<PD>::KW>* __restrict__ vkeys,
                       int* __restrict__ nbr, u64 max_entries) {
    after_previous_kernel();
    constexpr int KW = Cfg<PD>::KW;
    if (hdr->status != 0) return;
    resolve_entries(hdr, list_ref, vid);
    const u32 M = hdr->num_vertices;
    const u64 items = (u64)M * (PD + 1);
    for (u64 e = (u64)blockIdx.x * blockDim.x + threadIdx.x; e < items; e += (u64)gridDim.x * blockDim.x) {
        const u32 v = (u32)(e / (PD + 1));
        const int a = (int)(e - (u64)v * (PD + 1));
        const Key<KW> k = vkeys[v];
        Key<KW> nk;
#pragma unroll
        for (int j = 0; j < KW; j++) nk.w[j] = 0;
#pragma unroll
        for (int i = 0; i < PD; i++) key_set<KW>(nk, i, (u16)(key_get<KW>(k, i) + ((i == a) ? -PD : 1)));
        key_set<KW>(nk, PD, key_get<KW>(k, PD));
        u64 s;
        if (!direct_slot<PD>(d, nk, s)) continue;
        const u32 o = table[s];
        if (o == DIRECT_EMPTY) continue;
        const u32 u = o & ~VERTEX_FLAG;
        nbr[((u64)a * max_entries + v) * 2] = (int)u;
        nbr[((u64)a * max_entries + u) * 2 + 1] = (int)v;
    }
}

}  // namespace pl
