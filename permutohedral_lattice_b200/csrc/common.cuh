// Shared definitions of the lattice kernels: geometry of a call, workspace header and layout, packed
// vertex keys and their hashes, tile addressing, vector reductions and asynchronous-copy helpers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
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
    // T = double calls: the same three in double
    double spatial_std_d, feature_std_d;
    double scale_d[MAX_PD];
};

struct Header {   // first 256 bytes of the workspace
    u32 num_entries;
    u32 num_vertices;
    u32 status;
    u32 table_log2;
    u32 absmax_bits;   // deterministic mode: bit pattern of max |input| (non-negative floats order as integers)
    u32 direct;        // 1: vertices were found by direct indexing (spatial-only call), 0: through the hash table
    u32 capacity;      // the max_entries the workspace was laid out for (written by build_tiles)
    u32 sorted;        // 1: the lattice was built for reuse and holds every tile's splats sorted by entry
    u32 pad[56];
};

struct Layout {   // byte offsets into the workspace
    size_t tile_info, rec, rec_w, srec, list_keys, list_ref, vid, vkeys, table, nbr, v0, v1, v64, total;
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
    // The tile's splats sorted by entry, as build_tiles leaves them for the splat kernels: cut into windows
    // of WL splats, each followed by one spare 8-byte word (lanes that walk neighbouring windows in step then
    // read words an odd number of 8-byte words apart: no shared-memory bank collisions), SREC words per tile
    // (even: the list moves by bulk copies, whose sizes are multiples of 16 bytes).
    static constexpr int WL = 8 * (PD + 1);
    static constexpr int SREC = (SPLATS + SPLATS / WL + 1 + 1) & ~1;
    __host__ __device__ static constexpr int srec_slot(int pos) { return pos + pos / WL; }
    // build_tiles assembles that list in the memory of its key list, which is therefore at least as large
    static constexpr size_t BUILD_KEYS = sizeof(Key<KW>) * SPLATS > sizeof(uint2) * SREC ? sizeof(Key<KW>) * SPLATS
                                                                                        : sizeof(uint2) * SREC;
    static constexpr size_t BUILD_SMEM = BUILD_KEYS + sizeof(int) * LS + sizeof(u16) * SPLATS;
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

// Key read straight from L2 (no L1): for data that another CTA of the SAME launch may have written.
template <int KW>
__device__ __forceinline__ Key<KW> load_key_l2(const Key<KW>* p) {
    Key<KW> k;
    const unsigned long long* w = reinterpret_cast<const unsigned long long*>(p);
#pragma unroll
    for (int j = 0; j < KW; j++) k.w[j] = __ldcg(w + j);
    return k;
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

// T = double: the reference's expressions as they stand (int converted to double, IEEE divisions).
template <int PD>
__device__ __forceinline__ void load_features(const Geom& g, const double* __restrict__ positions,
                                              const double* __restrict__ reference, int item, int pix, int o,
                                              int y, int x, double* f) {
    if (g.from_positions) {
        const double* p = positions + ((size_t)item * g.n + pix) * PD;
#pragma unroll
        for (int i = 0; i < PD; i++) f[i] = __ldg(p + i);
    } else {
        const double* ref = reference + ((size_t)item * g.n + pix) * g.R;
        int rest = o;
#pragma unroll
        for (int i = PD - 1; i >= 0; i--) {
            if (i >= g.n_sdims) {
                f[i] = __ddiv_rn(__ldg(ref + (i - g.n_sdims)), g.feature_std_d);
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
                f[i] = __ddiv_rn((double)c, g.spatial_std_d);
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

// A call that failed on the device (status word set by an earlier launch) must not leave bytes that
// could pass for a result: the slice stage then fills the tile's output rows with NaN and returns.
template <typename T>
__device__ __forceinline__ void poison_tile_output(const Geom& g, T* __restrict__ output, int channels) {
    const TilePos tpos = this_tile(g);
    int item, pix;
    if (!tile_point(g, tpos, threadIdx.x, item, pix)) return;
    T* row = output + ((size_t)item * g.n + pix) * channels;
    const T nan = (T)__int_as_float(0x7FC00000);
    for (int j = 0; j < channels; j++) row[j] = nan;
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
__device__ __forceinline__ void red_add_f64(double* addr, double a) {
    asm volatile("red.global.add.f64 [%0], %1;" ::"l"(addr), "d"(a) : "memory");
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

// First statement of every kernel of a filter call.  A kernel launched with programmatic stream serialisation
// may become resident while the kernel before it in the stream is still draining: the first instruction waits
// until that kernel has finished and its writes are visible, the second lets the kernel AFTER this one become
// resident in its turn (its CTAs are scheduled once every CTA of this grid has got here).  Every kernel waits
// before it reads anything, so "the kernel before has finished" implies that all earlier ones have.  The release
// comes after the wait on purpose: released first, a waiting kernel lets the one after it wait beside it, and
// two kernels' worth of waiting CTAs on the SMs slowed a long-running tile kernel by a quarter (pd = 16).
// Both instructions do nothing in a plain launch.
__device__ __forceinline__ void after_previous_kernel() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// The two halves for kernels whose grid runs in several waves (the tile kernels): they let the next kernel
// start only when their own work is nearly done.  Released at their start, the next kernel's CTAs sat on the
// SMs beside the tile kernel's later waves and slowed them (measured: a call 15 % slower).
__device__ __forceinline__ void wait_for_previous_kernel() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void let_next_kernel_start() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Developer aid, compiled only with -DPL_PHASE_CLOCKS: cycles that thread 0 of every CTA spends between
// marks, summed per kernel and phase (read back with pl_debug_phase_cycles).  Off in the shipped build.
#ifdef PL_PHASE_CLOCKS
__device__ unsigned long long g_phase_cycles[8][16];
struct PhaseClock {
    long long t;
    int k, i;
    __device__ __forceinline__ PhaseClock(int kernel) : k(kernel), i(0) { t = clock64(); }
    __device__ __forceinline__ void mark(bool sync = false) {
        if (sync) __syncthreads();
        if (threadIdx.x == 0) {
            const long long n = clock64();
            atomicAdd(&g_phase_cycles[k][i], (unsigned long long)(n - t));
            t = n;
        }
        i++;
    }
};
#else
struct PhaseClock {
    __device__ __forceinline__ PhaseClock(int) {}
    __device__ __forceinline__ void mark(bool = false) {}
};
#endif

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

}  // namespace pl
