// B200 (sm_100a) permutohedral-lattice filter: kernels and the C ABI of include/pl_lattice.h.
//
// Pipeline of one call (whole batch in every launch, nothing synchronises with the host):
//
//   build_tiles     one CTA per tile of TP points: features -> enclosing simplex -> pd+1 vertex keys
//                   per point; the tile's keys are de-duplicated in a shared-memory hash; the
//                   distinct keys become a contiguous run of "entries" in a global list and every
//                   splat records the 16-bit index of its entry inside the tile.
//   clear_table     sizes the global hash table from the entry count (on the device) and clears it.
//   insert_entries  one CAS per entry into the table; the first entry of a key owns a new vertex.
//   link_vertices   entry -> vertex index; presets the neighbour table, zeroes the value rows.
//   link_neighbours the +-1 neighbours of every vertex along each of the pd+1 axes: one table lookup
//                   per vertex and axis fills both directions.
//   splat_tiles     one CTA per tile: barycentric weights recomputed, values accumulated per entry
//                   in shared memory, one row of global atomics per entry.
//   blur_axis       pd+1 launches: V'[v] = (V[n1] + 2 V[v] + V[n2]) / 4, Jacobi, ping-pong buffers.
//   slice_tiles     one CTA per tile: the tile's vertex rows staged in shared memory, each point
//                   interpolates, divides by the homogeneous channel and writes its output row.
//
// A table slot is one 64-bit word (32-bit hash tag | index of the owning entry); full keys are
// compared through the entry list, which a previous launch has completely written, so there are no
// locks, no waiting and no duplicate vertices.  All device loops are bounded.
#include <cuda_runtime.h>
#include <cmath>
#include <mutex>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/pl_lattice.h"
#include "simplex.cuh"

namespace pl {

typedef unsigned long long u64;
typedef unsigned int u32;
typedef unsigned short u16;

constexpr u64 EMPTY_SLOT = ~0ull;
constexpr int MAX_SDIMS = 8;
constexpr int MAX_PD = 16;

// ---------------------------------------------------------------------------------------------
// Geometry of a call: how points map to tiles and how features are produced.
// ---------------------------------------------------------------------------------------------
struct Geom {
    int batch, n;           // items, points per item
    int W, H, outer;        // n = outer * H * W (W fastest)
    int TX, TY;             // tile = TY rows of TX points, TX * TY = TP
    int tiles_x, tiles_y, tiles_per_item, num_tiles;
    int tx_log2;            // TX is a power of two
    int grid3;              // 1: tile kernels run on a (tiles_x, tiles_y, batch * outer) grid
    int n_sdims, R;         // op path: spatial dims and reference channels (pd = n_sdims + R)
    int sdims[MAX_SDIMS];
    float spatial_std, feature_std;
    float spatial_rcp, feature_rcp;   // correctly rounded reciprocals of the two (host-computed)
    int rcp_div;            // 1: divide through the reciprocals (exact for these operands), 0: IEEE divide
    int from_positions;     // 1: features are read from a positions array
    float scale[MAX_PD];    // host-computed scale factors (double arithmetic rounded to float)
};

struct Header {   // first 256 bytes of the workspace
    u32 num_entries;
    u32 num_vertices;
    u32 status;
    u32 table_log2;
    u32 absmax_bits;   // deterministic mode: bit pattern of max |input| (non-negative floats order as integers)
    u32 pad[59];
};

struct Layout {   // byte offsets into the workspace
    size_t tile_info, rec, rec_w, list_keys, list_ref, vid, vowner, table, nbr, v0, v1, v64, total;
    u64 max_entries;   // capacity of entry- and vertex-indexed arrays
    u64 table_slots;   // allocated slots (power of two)
};

template <int KW>
struct alignas((KW % 2 == 0) ? 16 : 8) Key {
    u64 w[KW];
};

template <int PD>
struct Cfg {
    static constexpr int KW = (PD + 1 + 3) / 4;          // 16-bit fields: PD coordinates + item
    static constexpr int TP = (PD <= 8) ? 256 : 128;     // points per tile = threads per CTA
    static constexpr int SPLATS = TP * (PD + 1);
    static constexpr int LS = (5 * SPLATS <= 4 * 1024)   ? 1024
                              : (5 * SPLATS <= 4 * 2048) ? 2048
                              : (5 * SPLATS <= 4 * 4096) ? 4096
                              : (5 * SPLATS <= 4 * 8192) ? 8192
                                                         : 16384;   // shared hash slots (>= 1.25 * SPLATS)
    static constexpr size_t BUILD_SMEM = sizeof(Key<KW>) * SPLATS + sizeof(int) * LS + sizeof(u16) * SPLATS;
};

template <int KW>
__device__ __forceinline__ u64 hash_key(const Key<KW>& k) {
    u64 h = 0x9E3779B97F4A7C15ull;
#pragma unroll
    for (int j = 0; j < KW; j++) {
        h ^= k.w[j];
        h *= 0xFF51AFD7ED558CCDull;
        h ^= h >> 32;
    }
    h *= 0xC4CEB9FE1A85EC53ull;
    h ^= h >> 29;
    return h;
}

template <int KW>
__device__ __forceinline__ bool key_equal(const Key<KW>& a, const Key<KW>& b) {
    bool eq = true;
#pragma unroll
    for (int j = 0; j < KW; j++) eq = eq && (a.w[j] == b.w[j]);
    return eq;
}

// 16-bit field f of a key.  Fields 0..PD-1: lattice coordinates biased by 0x8000 (so that adding small
// offsets to a packed word never carries between fields); field PD: batch item.
template <int KW>
__device__ __forceinline__ void key_set(Key<KW>& k, int f, u16 v) {
    k.w[f >> 2] |= (u64)v << (16 * (f & 3));
}
template <int KW>
__device__ __forceinline__ u16 key_get(const Key<KW>& k, int f) {
    return (u16)(k.w[f >> 2] >> (16 * (f & 3)));
}

// 0x0001 in every coordinate field of key word j.
template <int PD>
__device__ __forceinline__ constexpr u64 coord_ones(int j) {
    u64 m = 0;
    for (int f = 4 * j; f < 4 * j + 4; f++)
        if (f < PD) m |= 1ull << (16 * (f & 3));
    return m;
}

// Cheap 32-bit hash for the per-tile shared-memory table (placement only).
template <int KW>
__device__ __forceinline__ u32 tile_hash(const Key<KW>& k) {
    u32 h = 0;
#pragma unroll
    for (int j = 0; j < KW; j++) {
        h = (h ^ (u32)k.w[j]) * 0x9E3779B1u;
        h = (h ^ (u32)(k.w[j] >> 32)) * 0x85EBCA77u;
    }
    h ^= h >> 15;
    h *= 0x2C1B3C6Du;
    return h ^ (h >> 13);
}

// Tile of this CTA.  Tile kernels run on a 3-D grid (tile column, tile row, item * outer + outer index)
// whenever that fits the grid limits, so no thread divides to find its tile; else on a 1-D grid.
struct TilePos {
    int tile, item, o, ty, tx;
};
__device__ __forceinline__ TilePos this_tile(const Geom& g) {
    TilePos t;
    if (g.grid3) {
        t.tx = blockIdx.x;
        t.ty = blockIdx.y;
        const int z = blockIdx.z;
        if (g.outer == 1) {
            t.item = z;
            t.o = 0;
        } else {
            t.item = z / g.outer;
            t.o = z - t.item * g.outer;
        }
        t.tile = (z * g.tiles_y + t.ty) * g.tiles_x + t.tx;
    } else {
        t.tile = blockIdx.x;
        t.item = t.tile / g.tiles_per_item;
        int r = t.tile - t.item * g.tiles_per_item;
        const int per_plane = g.tiles_x * g.tiles_y;
        t.o = r / per_plane;
        r -= t.o * per_plane;
        t.ty = r / g.tiles_x;
        t.tx = r - t.ty * g.tiles_x;
    }
    return t;
}

// Point handled by thread `tid` of the tile: item, point index inside the item, validity; the long
// form also gives the point's position (outer index, row, column).
__device__ __forceinline__ bool tile_point(const Geom& g, const TilePos& t, int tid, int& item, int& pix, int& o,
                                           int& y, int& x) {
    item = t.item;
    o = t.o;
    const int ly = tid >> g.tx_log2, lx = tid & (g.TX - 1);
    y = t.ty * g.TY + ly;
    x = t.tx * g.TX + lx;
    pix = (o * g.H + y) * g.W + x;
    return (y < g.H) && (x < g.W);
}
__device__ __forceinline__ bool tile_point(const Geom& g, const TilePos& t, int tid, int& item, int& pix) {
    int o, y, x;
    return tile_point(g, t, tid, item, pix, o, y, x);
}

// Feature vector of a point.  Op path: src/PermutohedralLatticeCPU.h:464-473 (coordinate of each
// spatial dimension as float divided by spatial_std, reference channel divided by feature_std; IEEE
// divisions, not reciprocal multiplies).  The last two spatial coordinates are the point's row and
// column in its tile grid; only deeper dimensions need the reference's divide-and-modulo.
// Positions path: a row of the positions array.
template <int PD>
__device__ __forceinline__ void load_features(const Geom& g, const float* __restrict__ positions,
                                              const float* __restrict__ reference, int item, int pix, int o,
                                              int y, int x, float* f) {
    if (g.from_positions) {
        const float* p = positions + ((size_t)item * g.n + pix) * PD;
#pragma unroll
        for (int i = 0; i < PD; i++) f[i] = __ldg(p + i);
    } else {
        const float* ref = reference + ((size_t)item * g.n + pix) * g.R;
        int rest = o;
#pragma unroll
        for (int i = PD - 1; i >= 0; i--) {
            if (i >= g.n_sdims) {
                const float a = __ldg(ref + (i - g.n_sdims));
                f[i] = g.rcp_div ? div_by_rcp(a, g.feature_std, g.feature_rcp) : PL_FDIV(a, g.feature_std);
            } else {
                int c;
                if (i == g.n_sdims - 1 && g.n_sdims >= 2) {
                    c = x;
                } else if (i == g.n_sdims - 2) {
                    c = y;
                } else if (g.n_sdims == 1) {
                    c = x;
                } else {
                    c = rest % g.sdims[i];
                    rest /= g.sdims[i];
                }
                const float a = small_int_to_float(c);
                f[i] = g.rcp_div ? div_by_rcp(a, g.spatial_std, g.spatial_rcp) : PL_FDIV(a, g.spatial_std);
            }
        }
    }
}

// Floats of a vertex row: vd padded to a multiple of 4 (16-byte rows).
__host__ __device__ __forceinline__ int padded_vd(int vd) { return (vd + 3) & ~3; }

// Status word of the call, read once per CTA so that every thread takes the same branch even while
// other CTAs of the same launch are setting error bits.
__device__ __forceinline__ bool call_failed(const Header* hdr) {
    __shared__ u32 status_s;
    if (threadIdx.x == 0) status_s = hdr->status;
    __syncthreads();
    return status_s != 0;
}

// ---------------------------------------------------------------------------------------------
// build_tiles
// ---------------------------------------------------------------------------------------------
template <int PD>
__global__ void __launch_bounds__(Cfg<PD>::TP)
build_tiles(Geom g, const float* __restrict__ positions, const float* __restrict__ reference,
            Header* hdr, int2* __restrict__ tile_info, u16* __restrict__ rec, float* __restrict__ rec_w,
            Key<Cfg<PD>::KW>* __restrict__ list_keys, u32 max_entries) {
    constexpr int KW = Cfg<PD>::KW, TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS, LS = Cfg<PD>::LS;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Key<KW>* keys_s = reinterpret_cast<Key<KW>*>(smem_raw);
    int* hslots = reinterpret_cast<int*>(smem_raw + sizeof(Key<KW>) * SPLATS);
    u16* lidx_s = reinterpret_cast<u16*>(smem_raw + sizeof(Key<KW>) * SPLATS + sizeof(int) * LS);
    __shared__ int nloc_s, base_s;

    const TilePos tpos = this_tile(g);
    const int tid = threadIdx.x, tile = tpos.tile;
    for (int i = tid; i < LS; i += TP) hslots[i] = -1;
    if (tid == 0) nloc_s = 0;

    int item, pix, po, py, px;
    const bool valid = tile_point(g, tpos, tid, item, pix, po, py, px);
    if (valid) {
        float f[PD];
        float w[PD + 1];
        load_features<PD>(g, positions, reference, item, pix, po, py, px, f);
        Simplex<PD> s;
        find_simplex<PD>(f, g.scale, s);
        barycentric<PD>(s, w);
        // the weights are final: store them now so the writes overlap the de-duplication below
        float* recw_tile = rec_w + (size_t)tile * SPLATS;
#pragma unroll
        for (int r = 0; r <= PD; r++) recw_tile[r * TP + tid] = w[r];
        // Remainder-r vertex: coordinate i = rem0_i + r - (PD+1) [rank_i > PD - r]
        // (src/PermutohedralLatticeCPU.h:297-304).  In packed form: start from the remainder-0 key,
        // then per step add one to every coordinate field and take PD+1 off the one coordinate whose
        // rank is PD - r + 1.
        Key<KW> k;
#pragma unroll
        for (int j = 0; j < KW; j++) k.w[j] = 0;
#pragma unroll
        for (int i = 0; i < PD; i++) key_set<KW>(k, i, (u16)(s.rem0[i] + 0x8000));
        key_set<KW>(k, PD, (u16)item);
        keys_s[tid] = k;
#pragma unroll
        for (int r = 1; r <= PD; r++) {
#pragma unroll
            for (int i = 0; i < PD; i++)
                k.w[i >> 2] -= (s.rank[i] == PD - r + 1) ? ((u64)(PD + 1) << (16 * (i & 3))) : 0ull;
#pragma unroll
            for (int j = 0; j < KW; j++) k.w[j] += coord_ones<PD>(j);
            keys_s[r * TP + tid] = k;
        }
    }
    __syncthreads();

    // de-duplicate: the first splat to claim a slot for a key represents it.  The first probes of all
    // PD+1 keys are issued together (independent shared-memory accesses); most keys resolve there,
    // the rest walk on one at a time.
    int rep[PD + 1];
    {
        u32 slot[PD + 1];
        int cand[PD + 1];
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            rep[r] = -1;
            slot[r] = 0;
            cand[r] = -1;
            if (valid) {
                slot[r] = tile_hash<KW>(keys_s[r * TP + tid]) & (LS - 1);
                cand[r] = hslots[slot[r]];
            }
        }
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            if (valid && cand[r] < 0) {
                cand[r] = atomicCAS(&hslots[slot[r]], -1, r * TP + tid);
                if (cand[r] < 0) rep[r] = r * TP + tid;
            }
        }
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            if (valid && rep[r] < 0 && key_equal<KW>(keys_s[cand[r]], keys_s[r * TP + tid])) rep[r] = cand[r];
        }
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            if (valid && rep[r] < 0) {
                const int me = r * TP + tid;
                const Key<KW> k = keys_s[me];
                u32 s = (slot[r] + 1) & (LS - 1);
                int found = -1;
                for (int it = 0; it < LS; it++) {
                    int o = hslots[s];
                    if (o < 0) {
                        o = atomicCAS(&hslots[s], -1, me);
                        if (o < 0) { found = me; break; }
                    }
                    if (key_equal<KW>(keys_s[o], k)) { found = o; break; }
                    s = (s + 1) & (LS - 1);
                }
                rep[r] = found;
            }
        }
    }
    __syncthreads();
    // number the tile's entries: one shared-memory atomic per warp and remainder, not per owner
#pragma unroll
    for (int r = 0; r <= PD; r++) {
        const bool own = valid && rep[r] == r * TP + tid;
        const unsigned owners = __ballot_sync(0xFFFFFFFFu, own);
        if (owners) {
            const int lane = tid & 31, leader = __ffs(owners) - 1;
            int first = 0;
            if (lane == leader) first = atomicAdd(&nloc_s, __popc(owners));
            first = __shfl_sync(0xFFFFFFFFu, first, leader);
            if (own) lidx_s[r * TP + tid] = (u16)(first + __popc(owners & ((1u << lane) - 1u)));
        }
    }
    __syncthreads();
    if (tid == 0) {
        int cnt = nloc_s;
        u32 base = atomicAdd(&hdr->num_entries, (u32)cnt);
        if ((u64)base + (u64)cnt > (u64)max_entries) {
            atomicOr(&hdr->status, 1u << PL_CAPACITY_EXCEEDED);
            base_s = -1;
            tile_info[tile] = make_int2(0, 0);
        } else {
            base_s = (int)base;
            tile_info[tile] = make_int2((int)base, cnt);
        }
    }
    __syncthreads();
    const int base = base_s;
    u16* rec_tile = rec + (size_t)tile * SPLATS;
#pragma unroll
    for (int r = 0; r <= PD; r++) {
        const int me = r * TP + tid;
        u16 l = 0;
        if (valid && rep[r] >= 0) {
            l = lidx_s[rep[r]];
            if (rep[r] == me && base >= 0) list_keys[(size_t)base + l] = keys_s[me];
        }
        rec_tile[me] = l;
    }
}

// ---------------------------------------------------------------------------------------------
// clear_table: table capacity = power of two >= 2 * entries (at least 1024), chosen on the device.
// ---------------------------------------------------------------------------------------------
__global__ void clear_table(Header* hdr, u64* __restrict__ table, u32 max_log2) {
    if (hdr->status != 0) return;
    u32 need = 2u * hdr->num_entries;
    u32 lg = 10;
    while (lg < max_log2 && (1ull << lg) < (u64)need) lg++;
    if (blockIdx.x == 0 && threadIdx.x == 0) hdr->table_log2 = lg;
    const u64 cap = 1ull << lg;
    for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i < cap; i += (u64)gridDim.x * blockDim.x)
        table[i] = EMPTY_SLOT;
}

// ---------------------------------------------------------------------------------------------
// insert_entries
// ---------------------------------------------------------------------------------------------
// Returns the index of the entry owning `k` in the table, or -1 if absent.
template <int KW>
__device__ __forceinline__ int table_find(const u64* __restrict__ table, u64 mask,
                                          const Key<KW>* __restrict__ list_keys, const Key<KW>& k) {
    const u64 h = hash_key<KW>(k);
    const u32 tag = (u32)(h >> 32);
    u64 s = h & mask;
    for (u64 it = 0; it <= mask; it++) {
        const u64 cur = table[s];
        if (cur == EMPTY_SLOT) return -1;
        if ((u32)(cur >> 32) == tag) {
            const u32 o = (u32)cur;
            if (key_equal<KW>(list_keys[o], k)) return (int)o;
        }
        s = (s + 1) & mask;
    }
    return -1;
}

template <int KW>
__global__ void __launch_bounds__(256)
insert_entries(Header* hdr, u64* __restrict__ table, const Key<KW>* __restrict__ list_keys,
               u32* __restrict__ list_ref, u32* __restrict__ vid, u32* __restrict__ vowner) {
    if (call_failed(hdr)) return;
    const u32 T = hdr->num_entries;
    const u64 mask = (1ull << hdr->table_log2) - 1;
    __shared__ u32 warp_cnt[8];
    __shared__ u32 block_base;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (u32 start = blockIdx.x * 256u; start < T; start += gridDim.x * 256u) {
        const u32 t = start + threadIdx.x;
        bool winner = false;
        if (t < T) {
            const Key<KW> k = list_keys[t];
            const u64 h = hash_key<KW>(k);
            const u32 tag = (u32)(h >> 32);
            const u64 mine = ((u64)tag << 32) | (u64)t;
            u64 s = h & mask;
            u32 owner = 0xFFFFFFFFu;
            for (u64 it = 0; it <= mask; it++) {
                u64 cur = table[s];
                if (cur == EMPTY_SLOT) {
                    cur = atomicCAS(&table[s], EMPTY_SLOT, mine);
                    if (cur == EMPTY_SLOT) { owner = t; winner = true; break; }
                }
                if ((u32)(cur >> 32) == tag) {
                    const u32 o = (u32)cur;
                    if (key_equal<KW>(list_keys[o], k)) { owner = o; break; }
                }
                s = (s + 1) & mask;
            }
            if (owner == 0xFFFFFFFFu) {
                atomicOr(&hdr->status, 1u << PL_INTERNAL_ERROR);
                owner = t;
            }
            list_ref[t] = owner;
        }
        // vertex indices: one atomic per CTA and chunk
        const u32 ballot = __ballot_sync(0xFFFFFFFFu, winner);
        if (lane == 0) warp_cnt[warp] = __popc(ballot);
        __syncthreads();
        if (threadIdx.x == 0) {
            u32 tot = 0;
#pragma unroll
            for (int w = 0; w < 8; w++) { u32 c = warp_cnt[w]; warp_cnt[w] = tot; tot += c; }
            block_base = tot ? atomicAdd(&hdr->num_vertices, tot) : 0u;
        }
        __syncthreads();
        if (winner) {
            const u32 v = block_base + warp_cnt[warp] + __popc(ballot & ((1u << lane) - 1u));
            vid[t] = v;
            vowner[v] = t;
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------
// link_vertices: entry -> vertex, neighbour table preset to "missing", zeroed value rows.
// link_neighbours: the +-1 neighbours of every vertex along each of the PD+1 lattice axes.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
link_vertices(Header* hdr, u32* __restrict__ list_ref, const u32* __restrict__ vid, int* __restrict__ nbr,
              float* __restrict__ v0, long long* __restrict__ v64, u64 max_entries, int pd, int vd) {
    if (hdr->status != 0) return;
    const u32 T = hdr->num_entries, M = hdr->num_vertices;
    const u64 gtid = (u64)blockIdx.x * blockDim.x + threadIdx.x;
    const u64 gsz = (u64)gridDim.x * blockDim.x;
    for (u64 t = gtid; t < T; t += gsz) list_ref[t] = vid[list_ref[t]];
    int2* nb = reinterpret_cast<int2*>(nbr);
    for (int a = 0; a <= pd; a++)
        for (u64 v = gtid; v < M; v += gsz) nb[(u64)a * max_entries + v] = make_int2(-1, -1);
    if (vd == 0) return;   // lattice built ahead of its use: rows are zeroed by each apply
    const u64 cells = (u64)M * padded_vd(vd);
    if (v64) {
        for (u64 e = gtid; e < cells; e += gsz) v64[e] = 0;
    } else {
        for (u64 e = gtid; e < cells; e += gsz) v0[e] = 0.f;
    }
}

// One table lookup per (vertex v, axis a): the neighbour u whose key is v's key with every stored
// coordinate +1, except coordinate a which moves by -PD (along axis PD no stored coordinate is
// special; src/PermutohedralLatticeCPU.h:381-388).  Then u is v's "+" neighbour and v is u's "-"
// neighbour, so the second lookup of the reference is not needed.
template <int PD>
__global__ void __launch_bounds__(256)
link_neighbours(const Header* hdr, const u64* __restrict__ table,
                const Key<Cfg<PD>::KW>* __restrict__ list_keys, const u32* __restrict__ vid,
                const u32* __restrict__ vowner, int* __restrict__ nbr, u64 max_entries) {
    constexpr int KW = Cfg<PD>::KW;
    if (hdr->status != 0) return;
    const u32 M = hdr->num_vertices;
    const u64 mask = (1ull << hdr->table_log2) - 1;
    const u64 items = (u64)M * (PD + 1);
    for (u64 e = (u64)blockIdx.x * blockDim.x + threadIdx.x; e < items; e += (u64)gridDim.x * blockDim.x) {
        const u32 v = (u32)(e / (PD + 1));
        const int a = (int)(e - (u64)v * (PD + 1));
        const Key<KW> k = list_keys[vowner[v]];
        Key<KW> nk;
#pragma unroll
        for (int j = 0; j < KW; j++) nk.w[j] = 0;
#pragma unroll
        for (int i = 0; i < PD; i++) key_set<KW>(nk, i, (u16)(key_get<KW>(k, i) + ((i == a) ? -PD : 1)));
        key_set<KW>(nk, PD, key_get<KW>(k, PD));
        const int o = table_find<KW>(table, mask, list_keys, nk);
        if (o >= 0) {
            const u32 u = vid[o];
            nbr[((u64)a * max_entries + v) * 2] = (int)u;
            nbr[((u64)a * max_entries + u) * 2 + 1] = (int)v;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Value rows.  A vertex row holds vd floats padded to VP = a multiple of 4, so that rows are 16-byte
// aligned: every row access below is a float4, and a row of 22 channels covers exactly three
// 32-byte sectors.  Pad channels stay zero through splat and blur and are never sliced.
// ---------------------------------------------------------------------------------------------
// Vector reduction into global memory (sm_90+): one L2 operation per 16 bytes.
__device__ __forceinline__ void red_add_v4(float* addr, float4 v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z),
                 "f"(v.w)
                 : "memory");
}
__device__ __forceinline__ void red_add_v2(float* addr, float a, float b) {
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(addr), "f"(a), "f"(b) : "memory");
}
__device__ __forceinline__ void red_add_f32(float* addr, float a) {
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(a) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
    const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(sa), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// How a warp's lanes are spread over value rows: GS lanes (one float4 each) per row, PPW rows per
// warp instruction.  Rows wider than 32 quads are walked in chunks of 32 quads.
struct LaneMap {
    int gs, ppw, g, q0;
    bool active;
    __device__ __forceinline__ LaneMap(int qpr, int lane) {
        gs = qpr < 32 ? qpr : 32;
        ppw = 32 / gs;
        g = lane / gs;
        q0 = lane - g * gs;
        active = g < ppw;
    }
};

// ---------------------------------------------------------------------------------------------
// Bulk asynchronous copies (TMA engine, untiled form) with an mbarrier; every wait is bounded.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(u64* bar, unsigned count) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(bar);
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(u64* bar, unsigned bytes) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(bar);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(a), "r"(bytes) : "memory");
}
// global -> shared, 16-byte aligned addresses, size a multiple of 16 bytes
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, unsigned bytes, u64* bar) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    const unsigned a = (unsigned)__cvta_generic_to_shared(bar);
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(d),
                 "l"(gmem_src), "r"(bytes), "r"(a)
                 : "memory");
}
// Waits for phase `parity` of the barrier; gives up (returns false) after a bounded number of polls.
__device__ __forceinline__ bool mbar_wait(u64* bar, unsigned parity) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(bar);
    for (int it = 0; it < (1 << 20); it++) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(a), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
// shared -> global
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, unsigned bytes) {
    const unsigned sa = (unsigned)__cvta_generic_to_shared(smem_src);
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(sa), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_store_finish() {
    asm volatile("cp.async.bulk.commit_group;\n\tcp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void fence_async_proxy() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// First point and number of valid points of tile row `ly` (the run of points that is contiguous in
// memory); returns false if the row lies outside the item.
__device__ __forceinline__ bool tile_row(const Geom& g, const TilePos& tpos, int ly, int& first_row, int& count) {
    int item, pix;
    if (!tile_point(g, tpos, ly * g.TX, item, pix)) return false;
    const int x0 = pix % g.W;
    first_row = item * g.n + pix;
    count = min(g.TX, g.W - x0);
    return true;
}

// ---------------------------------------------------------------------------------------------
// splat_tiles: V[vertex] += sum over the tile's splats of weight * [input channels, 1].
// The splats of a tile are counting-sorted by entry in shared memory, then every entry's run is
// summed in registers, reading the tile's input rows from shared memory, and leaves the CTA as one
// vector reduction per 16 bytes.  No floating-point atomics in shared memory.
//
// Fast form (VD known at compile time): one THREAD per entry holds the whole row in registers;
// entries are handed to threads in order of run length so the lanes of a warp finish together; the
// input block arrives by bulk asynchronous copies when its rows are 16-byte aligned.
// Generic form (any vd): a group of lanes per entry, one float4 of channels per lane.
// ---------------------------------------------------------------------------------------------
template <int PD>
struct SplatCommon {
    static constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS, NW = TP / 32;

    // Counting sort of the tile's splats by entry.  On return (after the trailing barrier)
    // sorted_s[off_s[e] .. cur_s[e]) are entry e's splats as (point | entry << 16, weight bits);
    // cur_s must be zero for e < nloc on entry.  off_s may be nullptr when run starts are not needed.
    // WL > 0 stores sorted position pos at slot(pos): the list is cut into windows of WL splats and
    // laid out step-major, so that threads walking neighbouring windows in step read neighbouring words.
    template <int WL>
    __device__ static __forceinline__ int slot(int pos) {
        if constexpr (WL == 0)
            return pos;
        else
            return (pos % WL) * (SPLATS / WL) + pos / WL;
    }

    template <int WL>
    __device__ static __forceinline__ void sort_splats(bool valid, const int* l, const float* w, int nloc,
                                                       uint2* sorted_s, int* cur_s, int* off_s, int* wsum_s) {
        const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
        if (valid) {
#pragma unroll
            for (int r = 0; r <= PD; r++) atomicAdd(&cur_s[l[r]], 1);
        }
        __syncthreads();
        int local[PD + 1];
        int sum = 0;
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            const int i = tid * (PD + 1) + r;
            local[r] = sum;
            sum += (i < nloc) ? cur_s[i] : 0;
        }
        int incl = sum;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int t = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if (lane >= d) incl += t;
        }
        if (lane == 31) wsum_s[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            const int v = (lane < NW) ? wsum_s[lane] : 0;
            int vi = v;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int t = __shfl_up_sync(0xFFFFFFFFu, vi, d);
                if (lane >= d) vi += t;
            }
            wsum_s[lane] = vi - v;
        }
        __syncthreads();
        const int excl = incl - sum + wsum_s[warp];
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            const int i = tid * (PD + 1) + r;
            if (i < nloc) {
                if (off_s) off_s[i] = excl + local[r];
                cur_s[i] = excl + local[r];
            }
        }
        __syncthreads();
        if (valid) {
#pragma unroll
            for (int r = 0; r <= PD; r++) {
                const int pos = atomicAdd(&cur_s[l[r]], 1);
                sorted_s[slot<WL>(pos)] = make_uint2((unsigned)tid | ((unsigned)l[r] << 16), __float_as_uint(w[r]));
            }
        }
        __syncthreads();
    }
};

template <int PD, int VD>
struct SplatFast {
    static constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS, C = VD - 1;
    static constexpr size_t IN_BYTES = ((sizeof(float) * TP * C + 15) / 16) * 16;
    static constexpr size_t BYTES = IN_BYTES + sizeof(uint2) * SPLATS + 2 * sizeof(int) * SPLATS + sizeof(int) * TP;
};

// Adds a row held in registers to vertex row `vrow` (VP floats, 16-byte aligned).
template <int VP>
__device__ __forceinline__ void flush_row(float* vrow, float* acc) {
#pragma unroll
    for (int q = 0; q < VP / 4; q++)
        red_add_v4(vrow + 4 * q, make_float4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]));
#pragma unroll
    for (int j = 0; j < VP; j++) acc[j] = 0.f;
}

template <int PD, int VD>
__global__ void __launch_bounds__(Cfg<PD>::TP)
splat_tiles_fast(Geom g, const float* __restrict__ input, Header* hdr, const int2* __restrict__ tile_info,
                 const u16* __restrict__ rec, const float* __restrict__ rec_w,
                 const u32* __restrict__ list_ref, float* __restrict__ v0, int bulk_ok) {
    constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS, C = VD - 1, VP = (VD + 3) & ~3;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* in_s = reinterpret_cast<float*>(smem_raw);                                       // [TP][C]
    uint2* sorted_s = reinterpret_cast<uint2*>(smem_raw + SplatFast<PD, VD>::IN_BYTES);     // [SPLATS]
    int* cur_s = reinterpret_cast<int*>(sorted_s + SPLATS);                                 // [SPLATS]
    int* prow_s = cur_s + SPLATS;                                                           // [TP]
    u32* vid_s = reinterpret_cast<u32*>(prow_s + TP);                                       // [SPLATS] entry -> vertex
    __shared__ int wsum_s[32];
    __shared__ __align__(8) u64 bar;
    if (call_failed(hdr)) return;
    const TilePos tpos = this_tile(g);
    const int tid = threadIdx.x, tile = tpos.tile;
    const int2 info = tile_info[tile];
    const int base = info.x, nloc = info.y;

    int item, pix;
    const bool valid = tile_point(g, tpos, tid, item, pix);
    prow_s[tid] = valid ? item * g.n + pix : -1;
    for (int i = tid; i < nloc; i += TP) {
        cur_s[i] = 0;
        vid_s[i] = list_ref[base + i];
    }
    if (bulk_ok && tid == 0) mbar_init(&bar, 1);
    const int nvalid = __syncthreads_count(valid);

    // stage the tile's input rows in shared memory, [point][channel] without padding: one bulk copy
    // per tile row, each issued by its own thread; thread 0 announces the byte total (nvalid points)
    if (bulk_ok) {
        if (tid == 0) mbar_expect_tx(&bar, (unsigned)nvalid * C * 4u);
        if (tid < g.TY) {
            int first, count;
            if (tile_row(g, tpos, tid, first, count))
                bulk_load(in_s + (size_t)tid * g.TX * C, input + (size_t)first * C, (unsigned)count * C * 4u, &bar);
        }
    } else {
        for (int k = tid; k < TP * C; k += TP) {
            const int p = k / C, j = k - p * C;
            const int row = prow_s[p];
            if (row >= 0) cp_async4(in_s + k, input + (size_t)row * C + j);
        }
    }

    float w[PD + 1];
    int l[PD + 1];
    const u16* rec_tile = rec + (size_t)tile * SPLATS;
    const float* recw_tile = rec_w + (size_t)tile * SPLATS;
#pragma unroll
    for (int r = 0; r <= PD; r++) {
        l[r] = valid ? rec_tile[r * TP + tid] : 0;
        w[r] = valid ? recw_tile[r * TP + tid] : 0.f;
    }
    SplatCommon<PD>::template sort_splats<PD + 1>(valid, l, w, nloc, sorted_s, cur_s, nullptr, wsum_s);

    if (bulk_ok) {
        if (!mbar_wait(&bar, 0)) {
            atomicOr(&hdr->status, 1u << PL_INTERNAL_ERROR);
            return;
        }
    } else {
        cp_async_wait_all();
        __syncthreads();
    }

    // Every thread sums a window of PD+1 consecutive sorted splats in registers; whenever the entry
    // changes, and at the end of the window, the partial row leaves as vector reductions.
    const int total = nvalid * (PD + 1);
    const int first = tid * (PD + 1);
    if (first >= total) return;
    float acc[VP];
#pragma unroll
    for (int j = 0; j < VP; j++) acc[j] = 0.f;
    using SC = SplatCommon<PD>;
    int cur = (int)(sorted_s[SC::template slot<PD + 1>(first)].x >> 16);
#pragma unroll
    for (int i = 0; i <= PD; i++) {
        if (first + i < total) {
            const uint2 pw = sorted_s[SC::template slot<PD + 1>(first + i)];
            const int e = (int)(pw.x >> 16);
            if (e != cur) {
                flush_row<VP>(v0 + (size_t)vid_s[cur] * VP, acc);
                cur = e;
            }
            const float wt = __uint_as_float(pw.y);
            const float* x = in_s + (pw.x & 0xFFFFu) * C;
#pragma unroll
            for (int j = 0; j < C; j++) acc[j] = PL_FADD(acc[j], PL_FMUL(wt, x[j]));
            acc[C] = PL_FADD(acc[C], wt);
        }
    }
    flush_row<VP>(v0 + (size_t)vid_s[cur] * VP, acc);
}

template <int PD, int VD, int GL>
__global__ void __launch_bounds__(Cfg<PD>::TP)
splat_tiles_group(Geom g, const float* __restrict__ input, Header* hdr, const int2* __restrict__ tile_info,
                 const u16* __restrict__ rec, const float* __restrict__ rec_w,
                 const u32* __restrict__ list_ref, float* __restrict__ v0, int bulk_ok) {
    constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS, C = VD - 1, VP = (VD + 3) & ~3;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* in_s = reinterpret_cast<float*>(smem_raw);                                       // [TP][C]
    uint2* sorted_s = reinterpret_cast<uint2*>(smem_raw + SplatFast<PD, VD>::IN_BYTES);     // [SPLATS]
    int* cur_s = reinterpret_cast<int*>(sorted_s + SPLATS);                                 // [SPLATS]
    int* prow_s = cur_s + SPLATS;                                                           // [TP]
    __shared__ int wsum_s[32];
    __shared__ __align__(8) u64 bar;
    if (call_failed(hdr)) return;
    const TilePos tpos = this_tile(g);
    const int tid = threadIdx.x, tile = tpos.tile;
    const int2 info = tile_info[tile];
    const int base = info.x, nloc = info.y;

    int item, pix;
    const bool valid = tile_point(g, tpos, tid, item, pix);
    prow_s[tid] = valid ? item * g.n + pix : -1;
    for (int i = tid; i < nloc; i += TP) cur_s[i] = 0;
    if (bulk_ok && tid == 0) mbar_init(&bar, 1);
    const int nvalid = __syncthreads_count(valid);

    // stage the tile's input rows in shared memory, [point][channel] without padding: one bulk copy
    // per tile row, each issued by its own thread; thread 0 announces the byte total (nvalid points)
    if (bulk_ok) {
        if (tid == 0) mbar_expect_tx(&bar, (unsigned)nvalid * C * 4u);
        if (tid < g.TY) {
            int first, count;
            if (tile_row(g, tpos, tid, first, count))
                bulk_load(in_s + (size_t)tid * g.TX * C, input + (size_t)first * C, (unsigned)count * C * 4u, &bar);
        }
    } else {
        for (int k = tid; k < TP * C; k += TP) {
            const int p = k / C, j = k - p * C;
            const int row = prow_s[p];
            if (row >= 0) cp_async4(in_s + k, input + (size_t)row * C + j);
        }
    }

    float w[PD + 1];
    int l[PD + 1];
    const u16* rec_tile = rec + (size_t)tile * SPLATS;
    const float* recw_tile = rec_w + (size_t)tile * SPLATS;
#pragma unroll
    for (int r = 0; r <= PD; r++) {
        l[r] = valid ? rec_tile[r * TP + tid] : 0;
        w[r] = valid ? recw_tile[r * TP + tid] : 0.f;
    }
    SplatCommon<PD>::template sort_splats<GL * (PD + 1)>(valid, l, w, nloc, sorted_s, cur_s, nullptr, wsum_s);

    if (bulk_ok) {
        if (!mbar_wait(&bar, 0)) {
            atomicOr(&hdr->status, 1u << PL_INTERNAL_ERROR);
            return;
        }
    } else {
        cp_async_wait_all();
        __syncthreads();
    }

    // GL lanes share a window of GL (PD+1) consecutive sorted splats.  A row is cut into pieces of
    // 32 / GL bytes; lane h of the group sums pieces h, h + GL, h + 2 GL, ...  Whenever the entry
    // changes, and at the end of the window, the partial row leaves as reductions: the GL lanes'
    // pieces of one step are neighbours in memory, so each group issues one 32-byte request per step.
    constexpr int PF = 8 / GL;                 // floats per piece: 4, 2 or 1
    constexpr int NP = VP / PF;                // pieces per row
    constexpr int NPL = (NP + GL - 1) / GL;    // pieces per lane
    constexpr int WL = GL * (PD + 1);
    using SC = SplatCommon<PD>;
    const int total = nvalid * (PD + 1);
    const int h = tid % GL, first = (tid / GL) * WL;
    if (first >= total) return;
    float acc[NPL * PF];
#pragma unroll
    for (int j = 0; j < NPL * PF; j++) acc[j] = 0.f;
    int cur = (int)(sorted_s[SC::template slot<WL>(first)].x >> 16);
    auto flush = [&](int entry) {
        float* vrow = v0 + (size_t)list_ref[base + entry] * VP + h * PF;
#pragma unroll
        for (int k = 0; k < NPL; k++) {
            if (h + GL * k < NP) {
                float* dst = vrow + GL * PF * k;
                if constexpr (PF == 4)
                    red_add_v4(dst, make_float4(acc[4 * k], acc[4 * k + 1], acc[4 * k + 2], acc[4 * k + 3]));
                else if constexpr (PF == 2)
                    red_add_v2(dst, acc[2 * k], acc[2 * k + 1]);
                else
                    red_add_f32(dst, acc[k]);
            }
        }
#pragma unroll
        for (int j = 0; j < NPL * PF; j++) acc[j] = 0.f;
    };
#pragma unroll 4
    for (int i = 0; i < WL; i++) {
        if (first + i < total) {
            const uint2 pw = sorted_s[SC::template slot<WL>(first + i)];
            const int e = (int)(pw.x >> 16);
            if (e != cur) {
                flush(cur);
                cur = e;
            }
            const float wt = __uint_as_float(pw.y);
            const float* x = in_s + (pw.x & 0xFFFFu) * C + h * PF;
#pragma unroll
            for (int k = 0; k < NPL; k++) {
#pragma unroll
                for (int c = 0; c < PF; c++) {
                    const int j = (h + GL * k) * PF + c;      // channel of this lane's slot
                    if (j < C)
                        acc[PF * k + c] = PL_FADD(acc[PF * k + c], PL_FMUL(wt, x[GL * PF * k + c]));
                    else if (j == C)
                        acc[PF * k + c] = PL_FADD(acc[PF * k + c], wt);
                }
            }
        }
    }
    flush(cur);
}

template <int PD>
struct SplatGeneric {
    static constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS;
    static size_t bytes(int vd) {
        return sizeof(float) * (size_t)TP * padded_vd(vd) + sizeof(uint2) * SPLATS + 2 * sizeof(int) * SPLATS +
               sizeof(int) * TP;
    }
};

template <int PD>
__global__ void __launch_bounds__(Cfg<PD>::TP)
splat_tiles_generic(Geom g, const float* __restrict__ input, Header* hdr, const int2* __restrict__ tile_info,
                    const u16* __restrict__ rec, const float* __restrict__ rec_w,
                    const u32* __restrict__ list_ref, float* __restrict__ v0, int vd) {
    constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS, NW = TP / 32;
    const int C = vd - 1, VP = padded_vd(vd), QPR = VP >> 2;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* in_s = reinterpret_cast<float*>(smem_raw);                       // [TP][VP]
    uint2* sorted_s = reinterpret_cast<uint2*>(in_s + (size_t)TP * VP);     // [SPLATS]
    int* cur_s = reinterpret_cast<int*>(sorted_s + SPLATS);                 // [SPLATS]
    int* off_s = cur_s + SPLATS;                                            // [SPLATS]
    int* prow_s = off_s + SPLATS;                                           // [TP]
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
    in_s[tid * VP + C] = 1.f;   // homogeneous channel, then padding
    for (int j = C + 1; j < VP; j++) in_s[tid * VP + j] = 0.f;
    __syncthreads();
    for (int k = tid; k < TP * C; k += TP) {
        const int p = k / C, j = k - p * C;
        const int row = prow_s[p];
        if (row >= 0) cp_async4(in_s + p * VP + j, input + (size_t)row * C + j);
    }
    float w[PD + 1];
    int l[PD + 1];
    const u16* rec_tile = rec + (size_t)tile * SPLATS;
    const float* recw_tile = rec_w + (size_t)tile * SPLATS;
#pragma unroll
    for (int r = 0; r <= PD; r++) {
        l[r] = valid ? rec_tile[r * TP + tid] : 0;
        w[r] = valid ? recw_tile[r * TP + tid] : 0.f;
    }
    SplatCommon<PD>::template sort_splats<0>(valid, l, w, nloc, sorted_s, cur_s, off_s, wsum_s);
    cp_async_wait_all();
    __syncthreads();

    const LaneMap lm(QPR, lane);
    if (!lm.active) return;
    const float4* in4 = reinterpret_cast<const float4*>(in_s);
    for (int e = warp * lm.ppw + lm.g; e < nloc; e += NW * lm.ppw) {
        const int beg = off_s[e], end = cur_s[e];
        float* vrow = v0 + (size_t)list_ref[base + e] * VP;
        for (int q = lm.q0; q < QPR; q += lm.gs) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int sidx = beg; sidx < end; sidx++) {
                const uint2 pw = sorted_s[sidx];
                const float wt = __uint_as_float(pw.y);
                const float4 x = in4[(pw.x & 0xFFFFu) * QPR + q];
                acc.x = PL_FADD(acc.x, PL_FMUL(wt, x.x));
                acc.y = PL_FADD(acc.y, PL_FMUL(wt, x.y));
                acc.z = PL_FADD(acc.z, PL_FMUL(wt, x.z));
                acc.w = PL_FADD(acc.w, PL_FMUL(wt, x.w));
            }
            red_add_v4(vrow + 4 * q, acc);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Deterministic splat (PL_MODE_DETERMINISTIC): the same sort-by-entry and segmented reduction, but
// every product weight * value is rounded once onto a fixed-point grid and summed as a 64-bit
// integer, in registers and in global memory.  Integer addition is associative, so the sums do not
// depend on the order in which splats, windows or tiles arrive: results are bitwise reproducible.
// Grid spacing: 2^-36 of the next power of two above max(|input|, 1), found by a first pass.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
absmax_kernel(const float* __restrict__ input, u64 count, Header* hdr) {
    u32 m = 0;
    for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (u64)gridDim.x * blockDim.x)
        m = max(m, __float_as_uint(fabsf(input[i])));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, d));
    if ((threadIdx.x & 31) == 0 && m) atomicMax(&hdr->absmax_bits, m);
}

// 2^(36 - e) with 2^e > max(|input|, 1); finite inputs only.
__device__ __forceinline__ double fixed_scale(const Header* hdr) {
    const u32 bits = max(hdr->absmax_bits, __float_as_uint(1.0f));
    const int e = (int)((bits >> 23) & 0xFF) - 127 + 1;
    return __longlong_as_double((long long)(1023 + 36 - e) << 52);
}

template <int PD>
struct SplatDet {
    static constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS;
    static size_t bytes(int vd) {
        return ((sizeof(float) * (size_t)TP * (vd - 1) + 15) / 16) * 16 + sizeof(uint2) * SPLATS +
               sizeof(int) * SPLATS + sizeof(int) * TP;
    }
};

template <int PD>
__global__ void __launch_bounds__(Cfg<PD>::TP)
splat_tiles_det(Geom g, const float* __restrict__ input, Header* hdr, const int2* __restrict__ tile_info,
                const u16* __restrict__ rec, const float* __restrict__ rec_w,
                const u32* __restrict__ list_ref, long long* __restrict__ v64, int vd) {
    constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS, NW = TP / 32;
    const int C = vd - 1, VP = padded_vd(vd);
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* in_s = reinterpret_cast<float*>(smem_raw);                                                // [TP][C]
    uint2* sorted_s = reinterpret_cast<uint2*>(smem_raw + ((sizeof(float) * (size_t)TP * C + 15) / 16) * 16);
    int* cur_s = reinterpret_cast<int*>(sorted_s + SPLATS);
    int* prow_s = cur_s + SPLATS;
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
    for (int k = tid; k < TP * C; k += TP) {
        const int p = k / C, j = k - p * C;
        const int row = prow_s[p];
        if (row >= 0) cp_async4(in_s + k, input + (size_t)row * C + j);
    }
    float w[PD + 1];
    int l[PD + 1];
    const u16* rec_tile = rec + (size_t)tile * SPLATS;
    const float* recw_tile = rec_w + (size_t)tile * SPLATS;
#pragma unroll
    for (int r = 0; r <= PD; r++) {
        l[r] = valid ? rec_tile[r * TP + tid] : 0;
        w[r] = valid ? recw_tile[r * TP + tid] : 0.f;
    }
    SplatCommon<PD>::template sort_splats<0>(valid, l, w, nloc, sorted_s, cur_s, nullptr, wsum_s);
    cp_async_wait_all();
    __syncthreads();

    // warp-uniform walk over a contiguous chunk of the sorted splats, lanes over channels
    const double scale = fixed_scale(hdr);
    const int total = nvalid * (PD + 1);
    const int chunk = (total + NW - 1) / NW;
    const int beg = warp * chunk, end = min(total, beg + chunk);
    if (beg >= end) return;
    for (int j0 = 0; j0 < vd; j0 += 32) {
        const int j = j0 + lane;
        long long acc = 0;
        int cur = (int)(sorted_s[beg].x >> 16);
        for (int sidx = beg; sidx < end; sidx++) {
            const uint2 pw = sorted_s[sidx];
            const int e = (int)(pw.x >> 16);
            if (e != cur) {
                if (j < vd && acc)
                    atomicAdd(reinterpret_cast<u64*>(v64 + (size_t)list_ref[base + cur] * VP + j), (u64)acc);
                acc = 0;
                cur = e;
            }
            if (j < vd) {
                const float wt = __uint_as_float(pw.y);
                const float prod = (j < C) ? PL_FMUL(wt, in_s[(pw.x & 0xFFFFu) * C + j]) : wt;
                acc += __double2ll_rn(PL_DMUL((double)prod, scale));
            }
        }
        if (j < vd && acc)
            atomicAdd(reinterpret_cast<u64*>(v64 + (size_t)list_ref[base + cur] * VP + j), (u64)acc);
    }
}

// fixed-point sums -> float rows
__global__ void __launch_bounds__(256)
convert_fixed(const Header* hdr, const long long* __restrict__ v64, float* __restrict__ v0, int vp) {
    if (hdr->status != 0) return;
    const double inv = 1.0 / fixed_scale(hdr);
    const u64 cells = (u64)hdr->num_vertices * vp;
    for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i < cells; i += (u64)gridDim.x * blockDim.x)
        v0[i] = (float)PL_DMUL(__ll2double_rn(v64[i]), inv);
}

// Start of an apply on an already built lattice: value rows (or fixed-point sums) back to zero.
__global__ void __launch_bounds__(256)
zero_rows(Header* hdr, float* __restrict__ v0, long long* __restrict__ v64, int vp) {
    if (hdr->status != 0) return;
    if (blockIdx.x == 0 && threadIdx.x == 0) hdr->absmax_bits = 0;
    const u64 cells = (u64)hdr->num_vertices * vp;
    const u64 gtid = (u64)blockIdx.x * blockDim.x + threadIdx.x, gsz = (u64)gridDim.x * blockDim.x;
    if (v64) {
        for (u64 e = gtid; e < cells; e += gsz) v64[e] = 0;
    } else {
        for (u64 e = gtid; e < cells; e += gsz) v0[e] = 0.f;
    }
}

// ---------------------------------------------------------------------------------------------
// blur_axis: one [1 2 1]/4 pass along lattice axis `axis` (src/PermutohedralLatticeCPU.h:403-405:
// the three products and their sum in double, one rounding to float).  One float4 per thread.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float mix3(float a, float b, float c) {
    return (float)PL_DADD(PL_DADD(PL_DMUL(0.25, (double)a), PL_DMUL(0.5, (double)b)),
                          PL_DMUL(0.25, (double)c));
}

__global__ void __launch_bounds__(256)
blur_axis(const Header* hdr, const int* __restrict__ nbr_axis, const float* __restrict__ src,
          float* __restrict__ dst, int qpr) {
    if (hdr->status != 0) return;
    const u32 M = hdr->num_vertices;
    const u64 items = (u64)M * qpr;
    const float4* __restrict__ s = reinterpret_cast<const float4*>(src);
    float4* __restrict__ d = reinterpret_cast<float4*>(dst);
    const int2* __restrict__ nb = reinterpret_cast<const int2*>(nbr_axis);
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    for (u64 e = (u64)blockIdx.x * blockDim.x + threadIdx.x; e < items;
         e += (u64)gridDim.x * blockDim.x) {
        const u32 v = (u32)(e / qpr);
        const int j = (int)(e - (u64)v * qpr);
        const int2 n = __ldg(nb + v);
        const float4 b = s[e];
        const float4 a = (n.x >= 0) ? s[(u64)n.x * qpr + j] : zero;
        const float4 c = (n.y >= 0) ? s[(u64)n.y * qpr + j] : zero;
        d[e] = make_float4(mix3(a.x, b.x, c.x), mix3(a.y, b.y, c.y), mix3(a.z, b.z, c.z),
                           mix3(a.w, b.w, c.w));
    }
}

// ---------------------------------------------------------------------------------------------
// slice_tiles (src/PermutohedralLatticeCPU.h:333-352: float multiply-then-add per remainder in
// ascending order, reciprocal of the homogeneous channel in double, one multiply per channel).
// The tile's vertex rows are staged once in shared memory.
//
// Fast form (VD known at compile time): one thread per point interpolates the whole row in
// registers (float4 reads of the cached rows, row stride padded against bank conflicts), the
// output block is assembled in shared memory and leaves by bulk asynchronous copies when its rows
// are 16-byte aligned.
// Generic form (any vd): a group of lanes per point, one float4 of channels per lane.
// ---------------------------------------------------------------------------------------------
template <int PD, int VD>
struct SliceFast {
    static constexpr int TP = Cfg<PD>::TP, C = VD - 1, VP = (VD + 3) & ~3;
    static constexpr int RS = VP + 4;   // words between cached rows: 16-byte aligned, spreads banks
    static constexpr size_t OUT_BYTES = ((sizeof(float) * TP * C + 15) / 16) * 16;
    // the output block reuses the space of the cached rows once every thread has read them
    __host__ __device__ static size_t region(int rows_cap) {
        const size_t rows = ((sizeof(float) * (size_t)rows_cap * RS + 15) / 16) * 16;
        return rows > OUT_BYTES ? rows : OUT_BYTES;
    }
    static size_t bytes(int rows_cap) { return region(rows_cap) + sizeof(int) * TP; }
};

template <int PD, int VD>
__global__ void __launch_bounds__(Cfg<PD>::TP, (Cfg<PD>::TP == 256) ? 5 : 8)
slice_tiles_fast(Geom g, float* __restrict__ output, const Header* hdr, const int2* __restrict__ tile_info,
                 const u16* __restrict__ rec, const float* __restrict__ rec_w,
                 const u32* __restrict__ list_ref, const float* __restrict__ vsrc, int rows_cap, int bulk_ok) {
    constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS, C = VD - 1, VP = (VD + 3) & ~3, QPR = VP / 4;
    constexpr int RS = SliceFast<PD, VD>::RS;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* rows_s = reinterpret_cast<float*>(smem_raw);                                         // [rows_cap][RS]
    float* out_s = reinterpret_cast<float*>(smem_raw);                                          // [TP][C], later
    int* prow_s = reinterpret_cast<int*>(smem_raw + SliceFast<PD, VD>::region(rows_cap));       // [TP]
    if (call_failed(hdr)) return;
    const TilePos tpos = this_tile(g);
    const int tid = threadIdx.x, tile = tpos.tile;
    const int2 info = tile_info[tile];
    const int base = info.x, cnt = info.y;
    const int nrows = min(cnt, rows_cap);
    const float4* v4 = reinterpret_cast<const float4*>(vsrc);
    for (int i = tid; i < nrows * QPR; i += TP) {
        const int lrow = i / QPR, q = i - lrow * QPR;
        cp_async16(rows_s + lrow * RS + 4 * q, v4 + (size_t)list_ref[base + lrow] * QPR + q);
    }
    int item, pix;
    const bool valid = tile_point(g, tpos, tid, item, pix);
    prow_s[tid] = valid ? item * g.n + pix : -1;
    float w[PD + 1];
    int l[PD + 1];
    const u16* rec_tile = rec + (size_t)tile * SPLATS;
    const float* recw_tile = rec_w + (size_t)tile * SPLATS;
#pragma unroll
    for (int r = 0; r <= PD; r++) {
        l[r] = valid ? rec_tile[r * TP + tid] : 0;
        w[r] = valid ? recw_tile[r * TP + tid] : 0.f;
    }
    cp_async_wait_all();
    __syncthreads();
    float acc[VP];
#pragma unroll
    for (int j = 0; j < VP; j++) acc[j] = 0.f;
    if (valid && cnt <= rows_cap) {
        // every row of the tile is cached (the usual case): plain shared-memory reads
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            const float4* row = reinterpret_cast<const float4*>(rows_s + l[r] * RS);
#pragma unroll
            for (int q = 0; q < QPR; q++) {
                const float4 x = row[q];
                acc[4 * q] = PL_FADD(acc[4 * q], PL_FMUL(w[r], x.x));
                acc[4 * q + 1] = PL_FADD(acc[4 * q + 1], PL_FMUL(w[r], x.y));
                acc[4 * q + 2] = PL_FADD(acc[4 * q + 2], PL_FMUL(w[r], x.z));
                acc[4 * q + 3] = PL_FADD(acc[4 * q + 3], PL_FMUL(w[r], x.w));
            }
        }
    } else if (valid) {
        // a tile with more entries than the cache holds: the rest comes straight from global memory
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            const float4* row = (l[r] < nrows) ? reinterpret_cast<const float4*>(rows_s + l[r] * RS)
                                               : v4 + (size_t)list_ref[base + l[r]] * QPR;
#pragma unroll
            for (int q = 0; q < QPR; q++) {
                const float4 x = row[q];
                acc[4 * q] = PL_FADD(acc[4 * q], PL_FMUL(w[r], x.x));
                acc[4 * q + 1] = PL_FADD(acc[4 * q + 1], PL_FMUL(w[r], x.y));
                acc[4 * q + 2] = PL_FADD(acc[4 * q + 2], PL_FMUL(w[r], x.z));
                acc[4 * q + 3] = PL_FADD(acc[4 * q + 3], PL_FMUL(w[r], x.w));
            }
        }
    }
    __syncthreads();   // every cached row has been read: the output block may overwrite them
    if (valid) {
        const float inv = (float)(1.0 / (double)acc[C]);
#pragma unroll
        for (int j = 0; j < C; j++) out_s[tid * C + j] = PL_FMUL(acc[j], inv);
    }
    if (bulk_ok) {
        fence_async_proxy();
        __syncthreads();
        if (tid < g.TY) {
            int first, count;
            if (tile_row(g, this_tile(g), tid, first, count))   // recomputed: keeps registers free above
                bulk_store(output + (size_t)first * C, out_s + (size_t)tid * g.TX * C, (unsigned)count * C * 4u);
            bulk_store_finish();
        }
    } else {
        __syncthreads();
        for (int k = tid; k < TP * C; k += TP) {
            const int p = k / C, j = k - p * C;
            const int row = prow_s[p];
            if (row >= 0) output[(size_t)row * C + j] = out_s[k];
        }
    }
}

template <int PD>
struct SliceCfg {
    static constexpr int PW = ((2 * (PD + 1) + 1 + 3) / 4) * 4;   // words of a point record
};

template <int PD>
__global__ void __launch_bounds__(Cfg<PD>::TP)
slice_tiles_generic(Geom g, float* __restrict__ output, const Header* hdr, const int2* __restrict__ tile_info,
                    const u16* __restrict__ rec, const float* __restrict__ rec_w,
                    const u32* __restrict__ list_ref, const float* __restrict__ vsrc, int vd, int rows_cap) {
    constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS, PW = SliceCfg<PD>::PW;
    const int C = vd - 1, VP = padded_vd(vd), QPR = VP >> 2;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float4* rows4 = reinterpret_cast<float4*>(smem_raw);                            // [rows_cap][QPR]
    float* prec_s = reinterpret_cast<float*>(rows4 + (size_t)rows_cap * QPR);       // [TP][PW]
    int* prow_s = reinterpret_cast<int*>(prec_s + (size_t)TP * PW);                 // [TP]
    if (call_failed(hdr)) return;
    const TilePos tpos = this_tile(g);
    const int tid = threadIdx.x, tile = tpos.tile, lane = tid & 31, warp = tid >> 5;
    const int2 info = tile_info[tile];
    const int base = info.x, cnt = info.y;
    const int nrows = min(cnt, rows_cap);
    const float4* v4 = reinterpret_cast<const float4*>(vsrc);
    for (int i = tid; i < nrows * QPR; i += TP) {
        const int lrow = i / QPR, q = i - lrow * QPR;
        cp_async16(rows4 + i, v4 + (size_t)list_ref[base + lrow] * QPR + q);
    }
    int item, pix;
    const bool valid = tile_point(g, tpos, tid, item, pix);
    prow_s[tid] = valid ? item * g.n + pix : -1;
    float w[PD + 1];
    int l[PD + 1];
    const u16* rec_tile = rec + (size_t)tile * SPLATS;
    const float* recw_tile = rec_w + (size_t)tile * SPLATS;
#pragma unroll
    for (int r = 0; r <= PD; r++) {
        l[r] = valid ? rec_tile[r * TP + tid] : 0;
        w[r] = valid ? recw_tile[r * TP + tid] : 0.f;
    }
    cp_async_wait_all();
    __syncthreads();
    if (valid) {
        const float* rows = reinterpret_cast<const float*>(rows4);
        float norm = 0.f;
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            const float hv = (l[r] < nrows) ? rows[l[r] * VP + C]
                                            : vsrc[(size_t)list_ref[base + l[r]] * VP + C];
            norm = PL_FADD(norm, PL_FMUL(w[r], hv));
        }
        float* pr = prec_s + tid * PW;
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            pr[r] = w[r];
            pr[PD + 2 + r] = __int_as_float(l[r]);
        }
        pr[PD + 1] = (float)(1.0 / (double)norm);
    }
    __syncthreads();

    const LaneMap lm(QPR, lane);
    if (!lm.active) return;
    for (int i = lm.g; i < 32; i += lm.ppw) {
        const int p = warp * 32 + i;
        const int row = prow_s[p];
        if (row < 0) continue;
        float pr[PW];
        const float4* pr4 = reinterpret_cast<const float4*>(prec_s + p * PW);
#pragma unroll
        for (int k = 0; k < PW / 4; k++) {
            const float4 t = pr4[k];
            pr[4 * k] = t.x; pr[4 * k + 1] = t.y; pr[4 * k + 2] = t.z; pr[4 * k + 3] = t.w;
        }
        const float inv = pr[PD + 1];
        const float4* rp[PD + 1];
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            const int lr = __float_as_int(pr[PD + 2 + r]);
            rp[r] = (lr < nrows) ? (rows4 + lr * QPR) : (v4 + (size_t)list_ref[base + lr] * QPR);
        }
        float* out_row = output + (size_t)row * C;
        for (int q = lm.q0; q < QPR; q += lm.gs) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int r = 0; r <= PD; r++) {
                const float4 x = rp[r][q];
                acc.x = PL_FADD(acc.x, PL_FMUL(pr[r], x.x));
                acc.y = PL_FADD(acc.y, PL_FMUL(pr[r], x.y));
                acc.z = PL_FADD(acc.z, PL_FMUL(pr[r], x.z));
                acc.w = PL_FADD(acc.w, PL_FMUL(pr[r], x.w));
            }
            const int j = 4 * q;
            if (j < C) out_row[j] = PL_FMUL(acc.x, inv);
            if (j + 1 < C) out_row[j + 1] = PL_FMUL(acc.y, inv);
            if (j + 2 < C) out_row[j + 2] = PL_FMUL(acc.z, inv);
            if (j + 3 < C) out_row[j + 3] = PL_FMUL(acc.w, inv);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// positions kernel (the standalone ComputeKernel functor) and lattice export
// ---------------------------------------------------------------------------------------------
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

template <int PD>
__global__ void __launch_bounds__(Cfg<PD>::TP)
export_points(Geom g, const Header* hdr, const int2* __restrict__ tile_info, const u16* __restrict__ rec,
              const float* __restrict__ rec_w, const u32* __restrict__ list_ref,
              int32_t* __restrict__ pixel_vertex, float* __restrict__ pixel_weight) {
    constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS;
    if (hdr->status != 0) return;
    const TilePos tpos = this_tile(g);
    const int tid = threadIdx.x, tile = tpos.tile;
    int item, pix;
    if (!tile_point(g, tpos, tid, item, pix)) return;
    const int base = tile_info[tile].x;
    const u16* rec_tile = rec + (size_t)tile * SPLATS;
    const float* recw_tile = rec_w + (size_t)tile * SPLATS;
    const size_t o = ((size_t)item * g.n + pix) * (PD + 1);
#pragma unroll
    for (int r = 0; r <= PD; r++) {
        if (pixel_vertex) pixel_vertex[o + r] = (int32_t)list_ref[base + rec_tile[r * TP + tid]];
        if (pixel_weight) pixel_weight[o + r] = recw_tile[r * TP + tid];
    }
}

template <int PD>
__global__ void export_vertices(const Header* hdr, const Key<Cfg<PD>::KW>* __restrict__ list_keys,
                                const u32* __restrict__ vowner, long long max_vertices,
                                int16_t* __restrict__ vertex_keys, int32_t* __restrict__ vertex_item) {
    constexpr int KW = Cfg<PD>::KW;
    if (hdr->status != 0) return;
    const u32 M = hdr->num_vertices;
    for (u64 v = (u64)blockIdx.x * blockDim.x + threadIdx.x; v < M && v < (u64)max_vertices;
         v += (u64)gridDim.x * blockDim.x) {
        const Key<KW> k = list_keys[vowner[v]];
        if (vertex_keys) {
#pragma unroll
            for (int i = 0; i < PD; i++) vertex_keys[v * PD + i] = (int16_t)(key_get<KW>(k, i) ^ 0x8000);
        }
        if (vertex_item) vertex_item[v] = (int32_t)key_get<KW>(k, PD);
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
static thread_local char g_cuda_error[256] = "";
// Stage-boundary events for the next filter call of this thread (pl_profile_next_call); consumed by it.
static thread_local cudaEvent_t* g_stage_events = nullptr;

static int cuda_fail(cudaError_t e, const char* where) {
    snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s", where, cudaGetErrorString(e));
    return PL_CUDA_ERROR;
}
#define PL_CUDA(call)                                   \
    do {                                                \
        cudaError_t e_ = (call);                        \
        if (e_ != cudaSuccess) return cuda_fail(e_, #call); \
    } while (0)

static size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

static int tp_of(int pd) { return pd <= 8 ? 256 : 128; }
static int kw_of(int pd) { return (pd + 1 + 3) / 4; }

static bool pd_supported(int pd) {
    return pd == 1 || pd == 2 || pd == 3 || pd == 4 || pd == 5 || pd == 6 || pd == 7 || pd == 8 ||
           pd == 16;
}

// src/PermutohedralLatticeCPU.h:194-217, T = float: double arithmetic rounded to float.
static void scale_factors(int pd, float* out) {
    float inv_std_dev = (float)((pd + 1) * sqrt(2.0 / 3));
    for (int i = 0; i < pd; i++)
        out[i] = (float)(1.0 / sqrt((double)((i + 1) * (i + 2))) * (double)inv_std_dev);
}

static int make_geom(Geom& g, int batch, int n, int pd, int n_sdims, const int* sdims, int R,
                     float spatial_std, float feature_std, bool from_positions) {
    memset(&g, 0, sizeof(g));
    g.batch = batch;
    g.n = n;
    g.from_positions = from_positions ? 1 : 0;
    g.n_sdims = n_sdims;
    g.R = R;
    g.spatial_std = spatial_std;
    g.feature_std = feature_std;
    // Division through a correctly rounded reciprocal and one fused correction gives the IEEE quotient
    // as long as nothing leaves the normal range; keep the plain divide for extreme sigmas.
    auto tame = [](float v) { return std::isfinite(v) && std::fabs(v) >= 1e-18f && std::fabs(v) <= 1e18f; };
    g.spatial_rcp = 1.0f / spatial_std;
    g.feature_rcp = 1.0f / feature_std;
    g.rcp_div = (tame(spatial_std) && tame(feature_std)) ? 1 : 0;
    const int tp = tp_of(pd);
    if (from_positions || n_sdims < 2) {
        g.W = n; g.H = 1; g.outer = 1;
        g.TX = tp; g.TY = 1;
    } else {
        g.W = sdims[n_sdims - 1];
        g.H = sdims[n_sdims - 2];
        g.outer = 1;
        for (int i = 0; i < n_sdims - 2; i++) g.outer *= sdims[i];
        g.TX = 16;
        while (g.TX > 1 && g.TX / 2 >= g.W) g.TX /= 2;   // narrow images: narrower, taller tiles
        g.TY = tp / g.TX;
    }
    for (int i = 0; i < n_sdims; i++) g.sdims[i] = sdims[i];
    g.tiles_x = (g.W + g.TX - 1) / g.TX;
    g.tiles_y = (g.H + g.TY - 1) / g.TY;
    long long per_item = (long long)g.tiles_x * g.tiles_y * g.outer;
    long long total = per_item * batch;
    if (total > 0x7FFFFFFFll) return PL_INVALID_ARGUMENT;
    g.tiles_per_item = (int)per_item;
    g.num_tiles = (int)total;
    g.tx_log2 = 0;
    while ((1 << g.tx_log2) < g.TX) g.tx_log2++;
    g.grid3 = (g.tiles_y <= 65535 && (long long)batch * g.outer <= 65535) ? 1 : 0;
    scale_factors(pd, g.scale);
    return PL_OK;
}

static int make_layout(Layout& L, const Geom& g, int pd, int vd, int64_t max_entries_arg) {
    const u64 S = (u64)g.batch * (u64)g.n * (u64)(pd + 1);
    if (S >= 0x7FFFFFF0ull) return PL_INVALID_ARGUMENT;
    u64 E = (max_entries_arg <= 0 || (u64)max_entries_arg > S) ? S : (u64)max_entries_arg;
    if (E < 1) E = 1;
    L.max_entries = E;
    u64 slots = 1024;
    while (slots < 2 * E) slots <<= 1;
    L.table_slots = slots;
    const size_t tile_splats = (size_t)tp_of(pd) * (pd + 1);
    size_t off = align_up(sizeof(Header));
    L.tile_info = off; off += align_up(sizeof(int2) * (size_t)g.num_tiles);
    L.rec = off;       off += align_up(sizeof(u16) * tile_splats * (size_t)g.num_tiles);
    L.rec_w = off;     off += align_up(sizeof(float) * tile_splats * (size_t)g.num_tiles);
    L.list_keys = off; off += align_up(sizeof(u64) * kw_of(pd) * E);
    L.list_ref = off;  off += align_up(sizeof(u32) * E);
    L.vid = off;       off += align_up(sizeof(u32) * E);
    L.vowner = off;    off += align_up(sizeof(u32) * E);
    L.table = off;     off += align_up(sizeof(u64) * slots);
    L.nbr = off;       off += align_up(sizeof(int) * 2 * (size_t)(pd + 1) * E);
    L.v0 = off;        off += align_up(sizeof(float) * (size_t)padded_vd(vd) * E);
    L.v1 = off;        off += align_up(sizeof(float) * (size_t)padded_vd(vd) * E);
    L.v64 = off;       off += align_up(sizeof(long long) * (size_t)padded_vd(vd) * E);   // deterministic mode sums
    L.total = off;
    return PL_OK;
}

// Launch grid of the tile kernels (see this_tile).
static dim3 tile_grid(const Geom& g) {
    if (g.grid3) return dim3((unsigned)g.tiles_x, (unsigned)g.tiles_y, (unsigned)(g.batch * g.outer));
    return dim3((unsigned)g.num_tiles, 1, 1);
}

static int g_num_sms = 0;
static int num_sms() {
    if (g_num_sms == 0) {
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
        g_num_sms = sms;
    }
    return g_num_sms;
}

// Rows of the per-tile shared-memory vertex-row cache of slice_tiles (48 KB of rows at most).
static int rows_cap_for(int pd, int vd) {
    const int splats = tp_of(pd) * (pd + 1);
    int cap = (48 * 1024) / (padded_vd(vd) * (int)sizeof(float));
    if (cap > splats) cap = splats;
    if (cap < 1) cap = 1;
    return cap;
}

// True when every contiguous run of a tile's points starts on a 16-byte boundary and has a size that is
// a multiple of 16 bytes in a [points][channels] float array at `ptr`: then the tile's block can move
// by bulk asynchronous copies.
static bool bulk_rows_ok(const Geom& g, const void* ptr, int channels) {
    const long long row_bytes = 4ll * channels;
    return ((uintptr_t)ptr % 16 == 0) && (row_bytes * g.W) % 16 == 0 && (row_bytes * g.TX) % 16 == 0 &&
           (row_bytes * g.n) % 16 == 0 && (row_bytes * g.TX * g.TY) < (1ll << 31);
}

// splat / slice for value dimension vd: the instantiation with vd fixed at compile time where there
// is one, else the generic one.
template <int PD, int VD>
static int launch_splat(const Geom& g, const float* input, Header* hdr, const int2* tile_info, const u16* rec,
                        const float* rec_w, const u32* list_ref, float* v0, int vd, cudaStream_t st) {
    if constexpr (VD > 8) {          // wide rows: a group of lanes per window, 32-byte reduction requests
        const size_t smem = SplatFast<PD, VD>::BYTES - sizeof(int) * Cfg<PD>::SPLATS;   // no vertex-id cache
        // four lanes per window measured best for 24-float rows (two and eight lanes are within 10 %)
        PL_CUDA(cudaFuncSetAttribute(splat_tiles_group<PD, VD, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)smem));
        splat_tiles_group<PD, VD, 4><<<tile_grid(g), Cfg<PD>::TP, smem, st>>>(
            g, input, hdr, tile_info, rec, rec_w, list_ref, v0, bulk_rows_ok(g, input, VD - 1) ? 1 : 0);
    } else if constexpr (VD > 0) {
        const size_t smem = SplatFast<PD, VD>::BYTES;
        PL_CUDA(cudaFuncSetAttribute(splat_tiles_fast<PD, VD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        splat_tiles_fast<PD, VD><<<tile_grid(g), Cfg<PD>::TP, smem, st>>>(
            g, input, hdr, tile_info, rec, rec_w, list_ref, v0, bulk_rows_ok(g, input, VD - 1) ? 1 : 0);
    } else {
        const size_t smem = SplatGeneric<PD>::bytes(vd);
        if (smem > 200 * 1024) return PL_UNSUPPORTED_DIMS;
        PL_CUDA(cudaFuncSetAttribute(splat_tiles_generic<PD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        splat_tiles_generic<PD><<<tile_grid(g), Cfg<PD>::TP, smem, st>>>(g, input, hdr, tile_info, rec, rec_w,
                                                                        list_ref, v0, vd);
    }
    return PL_OK;
}

template <int PD, int VD>
static int launch_slice(const Geom& g, float* output, const Header* hdr, const int2* tile_info, const u16* rec,
                        const float* rec_w, const u32* list_ref, const float* vsrc, int vd, cudaStream_t st) {
    if constexpr (VD > 0) {
        int rows_cap = (40 * 1024) / (SliceFast<PD, VD>::RS * 4);
        if (rows_cap > Cfg<PD>::SPLATS) rows_cap = Cfg<PD>::SPLATS;
        const size_t smem = SliceFast<PD, VD>::bytes(rows_cap);
        PL_CUDA(cudaFuncSetAttribute(slice_tiles_fast<PD, VD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        slice_tiles_fast<PD, VD><<<tile_grid(g), Cfg<PD>::TP, smem, st>>>(
            g, output, hdr, tile_info, rec, rec_w, list_ref, vsrc, rows_cap, bulk_rows_ok(g, output, VD - 1) ? 1 : 0);
    } else {
        const int rows_cap = rows_cap_for(PD, vd);
        const size_t fixed = sizeof(float) * Cfg<PD>::TP * SliceCfg<PD>::PW + sizeof(int) * Cfg<PD>::TP;
        const size_t smem = sizeof(float) * (size_t)rows_cap * padded_vd(vd) + fixed;
        if (smem > 200 * 1024) return PL_UNSUPPORTED_DIMS;
        PL_CUDA(cudaFuncSetAttribute(slice_tiles_generic<PD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        slice_tiles_generic<PD><<<tile_grid(g), Cfg<PD>::TP, smem, st>>>(g, output, hdr, tile_info, rec, rec_w,
                                                                        list_ref, vsrc, vd, rows_cap);
    }
    return PL_OK;
}

#define PL_DISPATCH_VD(FN, PD_, vd, ...)                                   \
    ((vd) == 22  ? FN<PD_, 22>(__VA_ARGS__)                                 \
     : (vd) == 4 ? FN<PD_, 4>(__VA_ARGS__)                                  \
     : (vd) == 3 ? FN<PD_, 3>(__VA_ARGS__)                                  \
     : (vd) == 2 ? FN<PD_, 2>(__VA_ARGS__)                                  \
                 : FN<PD_, 0>(__VA_ARGS__))

enum { PH_BUILD = 1, PH_APPLY = 2 };   // halves of a call: lattice structure / values through it

template <int PD>
static int run_filter(const Geom& g, float* output, const float* input, const float* positions,
                      const float* reference, int vd, int reverse, int mode, void* workspace,
                      const Layout& L, cudaStream_t st, int phases = PH_BUILD | PH_APPLY) {
    constexpr int KW = Cfg<PD>::KW, TP = Cfg<PD>::TP;
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    Header* hdr = reinterpret_cast<Header*>(ws);
    int2* tile_info = reinterpret_cast<int2*>(ws + L.tile_info);
    u16* rec = reinterpret_cast<u16*>(ws + L.rec);
    float* rec_w = reinterpret_cast<float*>(ws + L.rec_w);
    Key<KW>* list_keys = reinterpret_cast<Key<KW>*>(ws + L.list_keys);
    u32* list_ref = reinterpret_cast<u32*>(ws + L.list_ref);
    u32* vid = reinterpret_cast<u32*>(ws + L.vid);
    u32* vowner = reinterpret_cast<u32*>(ws + L.vowner);
    u64* table = reinterpret_cast<u64*>(ws + L.table);
    int* nbr = reinterpret_cast<int*>(ws + L.nbr);
    float* v0 = reinterpret_cast<float*>(ws + L.v0);
    float* v1 = reinterpret_cast<float*>(ws + L.v1);
    long long* v64 = (mode == PL_MODE_DETERMINISTIC) ? reinterpret_cast<long long*>(ws + L.v64) : nullptr;

    cudaEvent_t* ev = g_stage_events;
    g_stage_events = nullptr;
    if (ev) PL_CUDA(cudaEventRecord(ev[0], st));
    if (phases & PH_BUILD) PL_CUDA(cudaMemsetAsync(hdr, 0, sizeof(Header), st));
    if (g.num_tiles == 0) return PL_OK;

    // per device and cheap, so set on every call rather than cached
    PL_CUDA(cudaFuncSetAttribute(build_tiles<PD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)Cfg<PD>::BUILD_SMEM));
    const int sms = num_sms();
    const int wide = sms * 8;
    int table_log2 = 0;
    while ((1ull << table_log2) < L.table_slots) table_log2++;

    if (phases & PH_BUILD) {
        build_tiles<PD><<<tile_grid(g), TP, Cfg<PD>::BUILD_SMEM, st>>>(
            g, positions, reference, hdr, tile_info, rec, rec_w, list_keys, (u32)L.max_entries);
        if (ev) PL_CUDA(cudaEventRecord(ev[1], st));
        clear_table<<<wide, 256, 0, st>>>(hdr, table, (u32)table_log2);
        insert_entries<KW><<<wide, 256, 0, st>>>(hdr, table, list_keys, list_ref, vid, vowner);
        link_vertices<<<wide, 256, 0, st>>>(hdr, list_ref, vid, nbr, v0, v64, L.max_entries, PD,
                                            (phases & PH_APPLY) ? vd : 0);
        link_neighbours<PD><<<wide, 256, 0, st>>>(hdr, table, list_keys, vid, vowner, nbr, L.max_entries);
        if (ev) PL_CUDA(cudaEventRecord(ev[2], st));
    } else {
        if (ev) { PL_CUDA(cudaEventRecord(ev[1], st)); }
        zero_rows<<<wide, 256, 0, st>>>(hdr, v0, v64, padded_vd(vd));
        if (ev) { PL_CUDA(cudaEventRecord(ev[2], st)); }
    }
    if (!(phases & PH_APPLY)) {
        PL_CUDA(cudaGetLastError());
        return PL_OK;
    }
    int rc = PL_OK;
    if (v64) {
        const size_t smem = SplatDet<PD>::bytes(vd);
        if (smem > 200 * 1024) return PL_UNSUPPORTED_DIMS;
        PL_CUDA(cudaFuncSetAttribute(splat_tiles_det<PD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        absmax_kernel<<<wide, 256, 0, st>>>(input, (u64)g.batch * g.n * (vd - 1), hdr);
        splat_tiles_det<PD><<<tile_grid(g), TP, smem, st>>>(g, input, hdr, tile_info, rec, rec_w, list_ref, v64, vd);
        convert_fixed<<<wide, 256, 0, st>>>(hdr, v64, v0, padded_vd(vd));
    } else {
        rc = PL_DISPATCH_VD(launch_splat, PD, vd, g, input, hdr, tile_info, rec, rec_w, list_ref, v0, vd, st);
    }
    if (rc != PL_OK) return rc;
    if (ev) PL_CUDA(cudaEventRecord(ev[3], st));
    float* src = v0;
    float* dst = v1;
    const int qpr = padded_vd(vd) / 4;
    for (int step = 0; step <= PD; step++) {
        const int axis = reverse ? PD - step : step;
        const int* nb = nbr + (size_t)axis * L.max_entries * 2;
        blur_axis<<<wide, 256, 0, st>>>(hdr, nb, src, dst, qpr);
        float* tmp = src; src = dst; dst = tmp;
    }
    if (ev) PL_CUDA(cudaEventRecord(ev[4], st));
    rc = PL_DISPATCH_VD(launch_slice, PD, vd, g, output, hdr, tile_info, rec, rec_w, list_ref, src, vd, st);
    if (rc != PL_OK) return rc;
    if (ev) PL_CUDA(cudaEventRecord(ev[5], st));
    PL_CUDA(cudaGetLastError());
    return PL_OK;
}

template <int PD>
static int run_export(const Geom& g, const float* positions, const float* reference, const void* workspace,
                      const Layout& L, long long max_vertices, int16_t* vertex_keys,
                      int32_t* vertex_item, int32_t* pixel_vertex, float* pixel_weight,
                      cudaStream_t st) {
    constexpr int KW = Cfg<PD>::KW, TP = Cfg<PD>::TP;
    const unsigned char* ws = static_cast<const unsigned char*>(workspace);
    const Header* hdr = reinterpret_cast<const Header*>(ws);
    if (g.num_tiles == 0) return PL_OK;
    if (pixel_vertex || pixel_weight)
        export_points<PD><<<tile_grid(g), TP, 0, st>>>(
            g, hdr, reinterpret_cast<const int2*>(ws + L.tile_info), reinterpret_cast<const u16*>(ws + L.rec),
            reinterpret_cast<const float*>(ws + L.rec_w), reinterpret_cast<const u32*>(ws + L.list_ref),
            pixel_vertex, pixel_weight);
    if (vertex_keys || vertex_item)
        export_vertices<PD><<<num_sms() * 4, 256, 0, st>>>(
            hdr, reinterpret_cast<const Key<KW>*>(ws + L.list_keys),
            reinterpret_cast<const u32*>(ws + L.vowner), max_vertices, vertex_keys, vertex_item);
    PL_CUDA(cudaGetLastError());
    return PL_OK;
}

#define PL_DISPATCH_PD(pd, CALL)            \
    switch (pd) {                           \
        case 1: return CALL(1);             \
        case 2: return CALL(2);             \
        case 3: return CALL(3);             \
        case 4: return CALL(4);             \
        case 5: return CALL(5);             \
        case 6: return CALL(6);             \
        case 7: return CALL(7);             \
        case 8: return CALL(8);             \
        case 16: return CALL(16);           \
        default: return PL_UNSUPPORTED_DIMS; \
    }

static int filter_common(const Geom& g, float* output, const float* input, const float* positions,
                         const float* reference, int pd, int vd, int reverse, void* workspace,
                         size_t workspace_bytes, int64_t max_entries, int mode, cudaStream_t st,
                         int phases = PH_BUILD | PH_APPLY) {
    if (mode != PL_MODE_ATOMIC && mode != PL_MODE_DETERMINISTIC) return PL_INVALID_ARGUMENT;
    Layout L;
    int rc = make_layout(L, g, pd, vd, max_entries);
    if (rc != PL_OK) return rc;
    if (workspace_bytes < L.total) return PL_WORKSPACE_TOO_SMALL;
#define CALL(P) run_filter<P>(g, output, input, positions, reference, vd, reverse, mode, workspace, L, st, phases)
    PL_DISPATCH_PD(pd, CALL)
#undef CALL
}

// Scratch of pl_lattice_filter_f32_noalloc: lives in the library image, one copy on every GPU that
// loads the library, until the process exits.  In host code the array's name is only a handle; the
// device address comes from cudaGetSymbolAddress, once per device, with that device current.
static __device__ __align__(256) unsigned char g_static_scratch[PL_STATIC_SCRATCH_BYTES];
constexpr int MAX_DEVICES = 64;
static void* g_static_scratch_addr[MAX_DEVICES] = {nullptr};
static std::mutex g_static_scratch_mutex;

static int static_scratch_of_current_device(void** out) {
    int dev = -1;
    PL_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) return PL_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (!g_static_scratch_addr[dev]) {
        void* addr = nullptr;
        PL_CUDA(cudaGetSymbolAddress(&addr, g_static_scratch));
        g_static_scratch_addr[dev] = addr;
    }
    *out = g_static_scratch_addr[dev];
    return PL_OK;
}

}  // namespace pl

using namespace pl;

extern "C" {

int pl_supported(int pd, int vd) { return pd_supported(pd) && vd >= 2 && vd <= 4096 ? 1 : 0; }

const char* pl_strerror(int status) {
    switch (status) {
        case PL_OK: return "ok";
        case PL_INVALID_ARGUMENT: return "invalid argument";
        case PL_UNSUPPORTED_DIMS: return "unsupported (pd, vd)";
        case PL_WORKSPACE_TOO_SMALL: return "workspace too small";
        case PL_CAPACITY_EXCEEDED: return "lattice entries exceed max_entries";
        case PL_CUDA_ERROR: return "CUDA error";
        case PL_INTERNAL_ERROR: return "internal error (bounded device loop gave up)";
    }
    return "unknown status";
}

const char* pl_last_cuda_error(void) { return g_cuda_error; }

int pl_workspace_bytes(int batch, int n, int pd, int vd, int n_spatial_dims, const int* spatial_dims,
                       int64_t max_entries, size_t* bytes) {
    if (!bytes || batch < 0 || n < 0 || batch > 65535) return PL_INVALID_ARGUMENT;
    if (!pl_supported(pd, vd)) return PL_UNSUPPORTED_DIMS;
    Geom g;
    int rc;
    if (spatial_dims) {
        if (n_spatial_dims < 1 || n_spatial_dims > MAX_SDIMS || n_spatial_dims > pd) return PL_INVALID_ARGUMENT;
        long long prod = 1;
        for (int i = 0; i < n_spatial_dims; i++) prod *= spatial_dims[i];
        if (prod != n) return PL_INVALID_ARGUMENT;
        rc = make_geom(g, batch, n, pd, n_spatial_dims, spatial_dims, pd - n_spatial_dims, 1.f, 1.f, false);
    } else {
        int one = n;
        rc = make_geom(g, batch, n, pd, 1, &one, pd - 1, 1.f, 1.f, true);
    }
    if (rc != PL_OK) return rc;
    Layout L;
    rc = make_layout(L, g, pd, vd, max_entries);
    if (rc != PL_OK) return rc;
    *bytes = L.total;
    return PL_OK;
}

int pl_compute_positions_f32(const float* reference, float* positions, int n,
                             int n_reference_channels, int n_spatial_dims, const int* spatial_dims,
                             float spatial_std, float feature_std, void* stream) {
    if (!positions || n < 0 || n_spatial_dims < 0 || n_spatial_dims > MAX_SDIMS ||
        n_reference_channels < 0 || (n_reference_channels > 0 && !reference) ||
        (n_spatial_dims > 0 && !spatial_dims))
        return PL_INVALID_ARGUMENT;
    if (n == 0) return PL_OK;
    Geom g;
    memset(&g, 0, sizeof(g));
    for (int i = 0; i < n_spatial_dims; i++) g.sdims[i] = spatial_dims[i];
    g.spatial_std = spatial_std;
    g.feature_std = feature_std;
    positions_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
        reference, positions, n, n_reference_channels, n_spatial_dims, g);
    PL_CUDA(cudaGetLastError());
    return PL_OK;
}

int pl_filter_f32(float* output, const float* input, const float* positions, int batch, int n,
                  int pd, int vd, int reverse, void* workspace, size_t workspace_bytes,
                  int64_t max_entries, int mode, void* stream) {
    if (batch < 0 || n < 0 || batch > 65535) return PL_INVALID_ARGUMENT;
    if (!pl_supported(pd, vd)) return PL_UNSUPPORTED_DIMS;
    if (batch == 0 || n == 0) return PL_OK;
    if (!output || !input || !positions || !workspace) return PL_INVALID_ARGUMENT;
    Geom g;
    int one = n;
    int rc = make_geom(g, batch, n, pd, 1, &one, pd - 1, 1.f, 1.f, true);
    if (rc != PL_OK) return rc;
    return filter_common(g, output, input, positions, nullptr, pd, vd, reverse, workspace,
                         workspace_bytes, max_entries, mode, (cudaStream_t)stream);
}

static int op_geom(Geom& g, int batch, int n_spatial_dims, const int* spatial_dims,
                   int n_reference_channels, int bilateral, float theta_alpha, float theta_beta,
                   float theta_gamma, int* pd_out, int* n_out) {
    if (batch < 0 || batch > 65535 || n_spatial_dims < 1 || n_spatial_dims > MAX_SDIMS || !spatial_dims ||
        n_reference_channels < 0)
        return PL_INVALID_ARGUMENT;
    long long n = 1;
    for (int i = 0; i < n_spatial_dims; i++) {
        if (spatial_dims[i] < 0) return PL_INVALID_ARGUMENT;
        n *= spatial_dims[i];
        if (n > 0x7FFFFFFFll) return PL_INVALID_ARGUMENT;
    }
    // src/LatticeFilterKernel.cpp:131-142
    const int R = bilateral ? n_reference_channels : 0;
    const int pd = n_spatial_dims + R;
    const float spatial_std = bilateral ? theta_alpha : theta_gamma;
    const float feature_std = bilateral ? theta_beta : -1.f;
    *pd_out = pd;
    *n_out = (int)n;
    if (!pd_supported(pd)) return PL_UNSUPPORTED_DIMS;
    return make_geom(g, batch, (int)n, pd, n_spatial_dims, spatial_dims, R, spatial_std, feature_std, false);
}

int pl_lattice_filter_f32(float* output, const float* input, const float* reference, int batch,
                          int n_spatial_dims, const int* spatial_dims, int n_input_channels,
                          int n_reference_channels, int bilateral, float theta_alpha,
                          float theta_beta, float theta_gamma, int reverse, void* workspace,
                          size_t workspace_bytes, int64_t max_entries, int mode, void* stream) {
    if (n_input_channels < 1) return PL_INVALID_ARGUMENT;
    Geom g;
    int pd = 0, n = 0;
    int rc = op_geom(g, batch, n_spatial_dims, spatial_dims, n_reference_channels, bilateral,
                     theta_alpha, theta_beta, theta_gamma, &pd, &n);
    if (rc != PL_OK) return rc;
    const int vd = n_input_channels + 1;
    if (!pl_supported(pd, vd)) return PL_UNSUPPORTED_DIMS;
    if (batch == 0 || n == 0) return PL_OK;
    if (!output || !input || !workspace || (g.R > 0 && !reference)) return PL_INVALID_ARGUMENT;
    return filter_common(g, output, input, nullptr, reference, pd, vd, reverse, workspace,
                         workspace_bytes, max_entries, mode, (cudaStream_t)stream);
}

int pl_lattice_filter_f32_noalloc(float* output, const float* input, const float* reference, int batch,
                                  int n_spatial_dims, const int* spatial_dims, int n_input_channels,
                                  int n_reference_channels, int bilateral, float theta_alpha,
                                  float theta_beta, float theta_gamma, int reverse, int64_t max_entries,
                                  void* stream) {
    if (n_input_channels < 1) return PL_INVALID_ARGUMENT;
    Geom g;
    int pd = 0, n = 0;
    int rc = op_geom(g, batch, n_spatial_dims, spatial_dims, n_reference_channels, bilateral, theta_alpha,
                     theta_beta, theta_gamma, &pd, &n);
    if (rc != PL_OK) return rc;
    const int vd = n_input_channels + 1;
    if (!pl_supported(pd, vd)) return PL_UNSUPPORTED_DIMS;
    if (batch == 0 || n == 0) return PL_OK;
    if (!output || !input || (g.R > 0 && !reference)) return PL_INVALID_ARGUMENT;
    // sizes beyond the built-in scratch are refused before anything is launched
    Layout L;
    rc = make_layout(L, g, pd, vd, max_entries);
    if (rc != PL_OK) return rc;
    if (L.total > (size_t)PL_STATIC_SCRATCH_BYTES) {
        snprintf(g_cuda_error, sizeof(g_cuda_error),
                 "pl_lattice_filter_f32_noalloc: this call needs %zu bytes of scratch, the built-in scratch holds %zu",
                 L.total, (size_t)PL_STATIC_SCRATCH_BYTES);
        return PL_WORKSPACE_TOO_SMALL;
    }
    void* scratch = nullptr;
    rc = static_scratch_of_current_device(&scratch);   // first call on a device: looks the address up
    if (rc != PL_OK) return rc;
    // the call itself zeroes the counters it needs (the 256-byte header) and the value rows it sums
    // into; everything else in the scratch is written before it is read
    return filter_common(g, output, input, nullptr, reference, pd, vd, reverse, scratch,
                         (size_t)PL_STATIC_SCRATCH_BYTES, max_entries, PL_MODE_ATOMIC, (cudaStream_t)stream);
}

int pl_lattice_build_f32(const float* reference, int batch, int n_spatial_dims, const int* spatial_dims,
                         int n_reference_channels, int bilateral, float theta_alpha, float theta_beta,
                         float theta_gamma, int max_value_dim, void* workspace, size_t workspace_bytes,
                         int64_t max_entries, void* stream) {
    Geom g;
    int pd = 0, n = 0;
    int rc = op_geom(g, batch, n_spatial_dims, spatial_dims, n_reference_channels, bilateral, theta_alpha,
                     theta_beta, theta_gamma, &pd, &n);
    if (rc != PL_OK) return rc;
    if (!pl_supported(pd, max_value_dim)) return PL_UNSUPPORTED_DIMS;
    if (batch == 0 || n == 0) return PL_OK;
    if (!workspace || (g.R > 0 && !reference)) return PL_INVALID_ARGUMENT;
    return filter_common(g, nullptr, nullptr, nullptr, reference, pd, max_value_dim, 0, workspace, workspace_bytes,
                         max_entries, PL_MODE_ATOMIC, (cudaStream_t)stream, PH_BUILD);
}

int pl_lattice_build_positions_f32(const float* positions, int batch, int n, int pd, int max_value_dim,
                                   void* workspace, size_t workspace_bytes, int64_t max_entries, void* stream) {
    if (batch < 0 || n < 0 || batch > 65535) return PL_INVALID_ARGUMENT;
    if (!pl_supported(pd, max_value_dim)) return PL_UNSUPPORTED_DIMS;
    if (batch == 0 || n == 0) return PL_OK;
    if (!positions || !workspace) return PL_INVALID_ARGUMENT;
    Geom g;
    int one = n;
    int rc = make_geom(g, batch, n, pd, 1, &one, pd - 1, 1.f, 1.f, true);
    if (rc != PL_OK) return rc;
    return filter_common(g, nullptr, nullptr, positions, nullptr, pd, max_value_dim, 0, workspace, workspace_bytes,
                         max_entries, PL_MODE_ATOMIC, (cudaStream_t)stream, PH_BUILD);
}

int pl_lattice_apply_f32(float* output, const float* input, int n_input_channels, int reverse, int mode, int batch,
                         int n, int pd, int n_spatial_dims, const int* spatial_dims, void* workspace,
                         size_t workspace_bytes, int64_t max_entries, void* stream) {
    if (n_input_channels < 1 || batch < 0 || n < 0 || batch > 65535) return PL_INVALID_ARGUMENT;
    const int vd = n_input_channels + 1;
    if (!pl_supported(pd, vd)) return PL_UNSUPPORTED_DIMS;
    if (batch == 0 || n == 0) return PL_OK;
    if (!output || !input || !workspace) return PL_INVALID_ARGUMENT;
    Geom g;
    int rc;
    if (spatial_dims) {
        if (n_spatial_dims < 1 || n_spatial_dims > MAX_SDIMS || n_spatial_dims > pd) return PL_INVALID_ARGUMENT;
        long long prod = 1;
        for (int i = 0; i < n_spatial_dims; i++) prod *= spatial_dims[i];
        if (prod != n) return PL_INVALID_ARGUMENT;
        rc = make_geom(g, batch, n, pd, n_spatial_dims, spatial_dims, pd - n_spatial_dims, 1.f, 1.f, false);
    } else {
        int one = n;
        rc = make_geom(g, batch, n, pd, 1, &one, pd - 1, 1.f, 1.f, true);
    }
    if (rc != PL_OK) return rc;
    return filter_common(g, output, input, nullptr, nullptr, pd, vd, reverse, workspace, workspace_bytes,
                         max_entries, mode, (cudaStream_t)stream, PH_APPLY);
}

int pl_profile_next_call(void** stage_events) {
    g_stage_events = reinterpret_cast<cudaEvent_t*>(stage_events);
    return PL_OK;
}

int pl_lattice_stats(const void* workspace, pl_stats* stats, void* stream) {
    if (!workspace || !stats) return PL_INVALID_ARGUMENT;
    Header h;
    PL_CUDA(cudaMemcpyAsync(&h, workspace, sizeof(Header), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    PL_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    stats->num_vertices = h.num_vertices;
    stats->num_entries = h.num_entries;
    stats->table_slots = (int64_t)1 << h.table_log2;
    stats->device_status = PL_OK;
    for (int code = PL_INVALID_ARGUMENT; code <= PL_INTERNAL_ERROR; code++)
        if (h.status & (1u << code)) stats->device_status = code;
    stats->reserved = 0;
    return PL_OK;
}

int pl_export_lattice(const void* workspace, const float* positions, const float* reference,
                      int batch, int n, int pd, int vd, int n_spatial_dims, const int* spatial_dims,
                      int n_reference_channels, float spatial_std, float feature_std,
                      int64_t max_entries, int64_t max_vertices, int16_t* vertex_keys,
                      int32_t* vertex_item, int32_t* pixel_vertex, float* pixel_weight,
                      void* stream) {
    if (!workspace || batch < 0 || n < 0 || batch > 65535) return PL_INVALID_ARGUMENT;
    if (!pl_supported(pd, vd)) return PL_UNSUPPORTED_DIMS;
    if (batch == 0 || n == 0) return PL_OK;
    Geom g;
    int rc;
    if (positions) {
        int one = n;
        rc = make_geom(g, batch, n, pd, 1, &one, pd - 1, 1.f, 1.f, true);
    } else {
        if (n_spatial_dims < 1 || n_spatial_dims > MAX_SDIMS || !spatial_dims ||
            n_spatial_dims + n_reference_channels != pd || (n_reference_channels > 0 && !reference))
            return PL_INVALID_ARGUMENT;
        rc = make_geom(g, batch, n, pd, n_spatial_dims, spatial_dims, n_reference_channels,
                       spatial_std, feature_std, false);
    }
    if (rc != PL_OK) return rc;
    Layout L;
    rc = make_layout(L, g, pd, vd, max_entries);
    if (rc != PL_OK) return rc;
#define CALL(P) run_export<P>(g, positions, reference, workspace, L, (long long)max_vertices, vertex_keys, \
                              vertex_item, pixel_vertex, pixel_weight, (cudaStream_t)stream)
    PL_DISPATCH_PD(pd, CALL)
#undef CALL
}

}  // extern "C"
