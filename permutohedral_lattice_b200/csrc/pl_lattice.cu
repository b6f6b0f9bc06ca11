// B200 (sm_100a) permutohedral-lattice filter: kernels and the C ABI of include/pl_lattice.h.
//
// Pipeline of one call (whole batch in every launch, nothing synchronises with the host):
//
//   build_tiles     one CTA per tile of TP points: features -> enclosing simplex -> pd+1 vertex keys
//                   per point; the tile's keys are de-duplicated in a shared-memory hash; the
//                   distinct keys become a contiguous run of "entries" in a global list and every
//                   splat records the 16-bit index of its entry inside the tile.
//   clear_table     sizes the global hash table from the entry count (on the device) and clears it.
//   insert_entries  one CAS per entry into the table; the first entry of a key owns a new vertex, whose
//                   neighbour slots and value row the same launch initialises.
//   link_neighbours entry -> vertex index; then the +-1 neighbours of every vertex along each of the
//                   pd+1 axes: one table lookup per vertex and axis fills both directions.
//   splat_tiles     one CTA per tile: input block staged in shared memory (bulk async copies), splats
//                   sorted by entry, runs summed in registers, vector reductions into the vertex rows.
//   blur_axis       pd+1 launches: V'[v] = (V[n1] + 2 V[v] + V[n2]) / 4, Jacobi, ping-pong buffers.
//   slice_tiles     one CTA per tile: the tile's vertex rows staged in shared memory, each point
//                   interpolates, divides by the homogeneous channel and writes its output row.
//
// A table slot is one 64-bit word (32-bit hash tag | index of the owning entry); full keys are
// compared through the entry list, which a previous launch has completely written, so there are no
// locks, no waiting and no duplicate vertices.  All device loops are bounded.
//
// Device code lives in the headers included below (one translation unit); this file holds the host
// side: geometry and workspace layout, launches, and the extern "C" entry points.
#include <cuda_runtime.h>
#include <atomic>
#include <cmath>
#include <mutex>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <utility>

#include "common.cuh"
#include "lattice_build.cuh"
#include "direct_index.cuh"
#include "splat.cuh"
#include "blur_slice.cuh"
#include "export.cuh"
#include "fp64.cuh"
#include "crf.cuh"

namespace pl {

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
static thread_local char g_cuda_error[256] = "";
// Stage-boundary events for the next filter call of this thread (pl_profile_next_call); consumed by it.
static thread_local cudaEvent_t* g_stage_events = nullptr;

// Kernel launches issued by the library since it was loaded (pl_launch_count): memsets and event
// records are not counted.
static std::atomic<unsigned long long> g_launches{0};
#define PL_COUNT_LAUNCHES(n) g_launches.fetch_add((n), std::memory_order_relaxed)

static int cuda_fail(cudaError_t e, const char* where) {
    snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s", where, cudaGetErrorString(e));
    return PL_CUDA_ERROR;
}
#define PL_CUDA(call)                                   \
    do {                                                \
        cudaError_t e_ = (call);                        \
        if (e_ != cudaSuccess) return cuda_fail(e_, #call); \
    } while (0)

// Kernel launch with the error check of every other runtime call.  overlap: with programmatic stream
// serialisation, i.e. the kernel may become resident while the kernel before it in the stream drains (it waits
// in after_previous_kernel() until that kernel has finished).
template <typename... Params, typename... Args>
static cudaError_t launch_kernel(bool overlap, void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr = {};
    if (overlap) {
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#define PL_LAUNCH(kernel, grid, block, smem, st, ...) \
    PL_CUDA(launch_kernel(false, kernel, dim3(grid), dim3(block), smem, st, __VA_ARGS__))
// Which launches overlap the tail of the kernel before them (bits of PL_OVERLAP), each measured on its own
// (B200, 16 items / 2 items of the dense-CRF workload, ms per forward + backward step, all others as chosen):
// the blur passes after one another 2.023 -> 2.007 / 0.353 -> 0.342; the slice after the last pass and the
// splat after link_neighbours -> 2.002 / 0.335; clear_table after build_tiles -> 1.993 / 0.331; insert_entries
// after clear_table -> 1.992 / 0.328 (small tables only, see run_filter).  Left plain because they measured
// slower at 16 items: link_neighbours
// after insert_entries (index stage 0.175 -> 0.181 ms; in small calls it gains or loses 0.5 %) and the first
// blur pass after the splat (2.09).
enum { OV_BLUR = 1, OV_INSERT = 2, OV_SPLAT = 4, OV_BLUR0 = 8, OV_SLICE = 16, OV_CLEAR = 32, OV_LINK = 64 };
#ifndef PL_OVERLAP
#define PL_OVERLAP (OV_BLUR | OV_INSERT | OV_SPLAT | OV_SLICE | OV_CLEAR)
#endif
#define PL_LAUNCH_AFTER(which, kernel, grid, block, smem, st, ...) \
    PL_CUDA(launch_kernel((PL_OVERLAP & (which)) != 0, kernel, dim3(grid), dim3(block), smem, st, __VA_ARGS__))

static size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

static int tp_of(int pd) { return pd <= 8 ? 256 : 128; }
static int kw_of(int pd) { return (pd + 1 + 3) / 4; }
// 8-byte words of a tile's sorted splat list (Cfg<PD>::SREC)
static int srec_words_of(int pd) {
    const int splats = tp_of(pd) * (pd + 1), wl = 8 * (pd + 1);
    return (splats + splats / wl + 1 + 1) & ~1;
}

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

// T = double: standard deviations and scale factors (src/PermutohedralLatticeCPU.h:194-217) in double.
static void set_geom_f64(Geom& g, int pd, double spatial_std, double feature_std) {
    g.spatial_std_d = spatial_std;
    g.feature_std_d = feature_std;
    const double inv_std_dev = (pd + 1) * sqrt(2.0 / 3);
    for (int i = 0; i < pd; i++) g.scale_d[i] = 1.0 / sqrt((double)((i + 1) * (i + 2))) * inv_std_dev;
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

// real_bytes: 4 for float calls, 8 for double calls (wider weights and value rows, no fixed-point sums).
// with_fixed_point: the workspace also holds the 64-bit sums of the deterministic mode (float calls only).
static int make_layout(Layout& L, const Geom& g, int pd, int vd, int64_t max_entries_arg, int real_bytes = 4,
                       bool with_fixed_point = false) {
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
    L.rec_w = off;     off += align_up((size_t)real_bytes * tile_splats * (size_t)g.num_tiles);
    L.srec = off;      // the splats of every tile sorted by entry (float calls: what their splat kernels walk)
    if (real_bytes == 4) off += align_up(sizeof(uint2) * (size_t)srec_words_of(pd) * (size_t)g.num_tiles);
    L.list_keys = off; off += align_up(sizeof(u64) * kw_of(pd) * E);
    L.list_ref = off;  off += align_up(sizeof(u32) * E);
    L.vid = off;       off += align_up(sizeof(u32) * E);
    L.vkeys = off;     off += align_up(sizeof(u64) * kw_of(pd) * E);
    L.table = off;     off += align_up(sizeof(u64) * slots);
    L.nbr = off;       off += align_up(sizeof(int) * 2 * (size_t)(pd + 1) * E);
    const size_t row_bytes = real_bytes == 8 ? sizeof(double) * (size_t)padded_vd_f64(vd)
                                             : sizeof(float) * (size_t)padded_vd(vd);
    L.v0 = off;        off += align_up(row_bytes * E);
    L.v1 = off;        off += align_up(row_bytes * E);
    L.v64 = off;       // deterministic mode sums (float calls only)
    if (real_bytes == 4 && with_fixed_point) off += align_up(sizeof(long long) * (size_t)padded_vd(vd) * E);
    L.total = off;
    return PL_OK;
}

// Developer switch (pl_debug_direct_index): 0 sends spatial-only calls through the hash table too.
static int g_direct_index_enabled = 1;

// The dense index of a spatial-only call (direct_bounds.h), if the call qualifies and the index fits the
// table region of the workspace (32-bit slots in the memory of the 64-bit hash slots).
static bool make_direct(Direct& d, const Geom& g, int pd, const Layout& L) {
    memset(&d, 0, sizeof(d));
    if (!g_direct_index_enabled || g.from_positions || g.R != 0 || pd != g.n_sdims) return false;
    return direct_bounds(d, pd, g.sdims, g.spatial_std, g.scale, g.batch, 2 * L.table_slots);
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

// cudaFuncSetAttribute is a driver call and its effect lasts as long as the context: the dynamic
// shared-memory limit (and carve-out preference) of a kernel is raised once per device, and again only
// when a later call needs more than any call before it.
constexpr int MAX_DEVICES = 64;
template <auto Kernel>
static int ensure_dynamic_smem(size_t bytes, bool max_carveout = false) {
    static std::atomic<size_t> granted[MAX_DEVICES];   // zero-initialised: nothing granted yet
    int dev = -1;
    PL_CUDA(cudaGetDevice(&dev));
    const bool cached = dev >= 0 && dev < MAX_DEVICES;
    if (cached && granted[dev].load(std::memory_order_acquire) >= bytes + 1) return PL_OK;
    PL_CUDA(cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    if (max_carveout)
        PL_CUDA(cudaFuncSetAttribute(Kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                     cudaSharedmemCarveoutMaxShared));
    if (cached) granted[dev].store(bytes + 1, std::memory_order_release);
    return PL_OK;
}
#define PL_TRY(call)                     \
    do {                                 \
        const int rc_ = (call);          \
        if (rc_ != PL_OK) return rc_;    \
    } while (0)

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
template <int PD, int VD, bool PRE>
static int launch_splat_as(const Geom& g, const float* input, Header* hdr, const int2* tile_info, const u16* rec,
                           const float* rec_w, const uint2* srec, const u32* list_ref, float* v0, int vd,
                           cudaStream_t st) {
    if constexpr (VD > 8 && VD <= 32) {   // wide rows: a quarter warp per window, conflict-free row reads
        using SR = SplatRows<PD, VD, PRE>;
        const size_t smem = SR::BYTES;
        // five CTAs per SM need nearly all of the SM's shared memory: ask for the largest carve-out
        PL_TRY((ensure_dynamic_smem<splat_tiles_rows<PD, VD, PRE>>(smem, true)));
        // bulk staging also needs 16-byte aligned landing zones inside the padded tile rows
        const bool bulk = bulk_rows_ok(g, input, VD - 1) && g.TX <= 16 && (g.TX * (SR::VP - (VD - 1))) % 4 == 0;
        PL_LAUNCH_AFTER(OV_SPLAT, (splat_tiles_rows<PD, VD, PRE>), tile_grid(g), Cfg<PD>::TP, smem, st, g, input, hdr, tile_info, rec, rec_w,
                                                                              srec, list_ref, v0, bulk ? 1 : 0);
    } else if constexpr (VD > 0) {
        const size_t smem = SplatFast<PD, VD, PRE>::BYTES;
        PL_TRY((ensure_dynamic_smem<splat_tiles_fast<PD, VD, PRE>>(smem)));
        PL_LAUNCH_AFTER(OV_SPLAT, (splat_tiles_fast<PD, VD, PRE>), tile_grid(g), Cfg<PD>::TP, smem, st, g, input, hdr, tile_info, rec, rec_w,
                                                                              srec, list_ref, v0, bulk_rows_ok(g, input, VD - 1) ? 1 : 0);
    } else {
        const size_t smem = SplatGeneric<PD>::bytes(vd);
        if (smem > 200 * 1024) return PL_UNSUPPORTED_DIMS;
        PL_TRY((ensure_dynamic_smem<splat_tiles_generic<PD>>(smem)));
        PL_LAUNCH_AFTER(OV_SPLAT, (splat_tiles_generic<PD>), tile_grid(g), Cfg<PD>::TP, smem, st, g, input, hdr, tile_info, rec, rec_w,
                                                                        list_ref, v0, vd);
    }
    return PL_OK;
}

// presorted: the lattice was built for reuse (build_tiles with SORTED) and holds its splats sorted in srec
template <int PD, int VD>
static int launch_splat(const Geom& g, const float* input, Header* hdr, const int2* tile_info, const u16* rec,
                        const float* rec_w, const uint2* srec, bool presorted, const u32* list_ref, float* v0, int vd,
                        cudaStream_t st) {
    return presorted ? launch_splat_as<PD, VD, true>(g, input, hdr, tile_info, rec, rec_w, srec, list_ref, v0, vd, st)
                     : launch_splat_as<PD, VD, false>(g, input, hdr, tile_info, rec, rec_w, srec, list_ref, v0, vd, st);
}

template <int PD, int VD>
static int launch_slice(const Geom& g, float* output, const Header* hdr, const int2* tile_info, const u16* rec,
                        const float* rec_w, const u32* list_ref, const float* vsrc, int vd, cudaStream_t st) {
    if constexpr (VD > 0) {
        int rows_cap = (40 * 1024) / (SliceFast<PD, VD>::RS * 4);
        if (rows_cap > Cfg<PD>::SPLATS) rows_cap = Cfg<PD>::SPLATS;
        const size_t smem = SliceFast<PD, VD>::bytes(rows_cap);
        PL_TRY((ensure_dynamic_smem<slice_tiles_fast<PD, VD>>(smem)));
        PL_LAUNCH_AFTER(OV_SLICE, (slice_tiles_fast<PD, VD>), tile_grid(g), Cfg<PD>::TP, smem, st, g, output, hdr, tile_info, rec, rec_w, list_ref, vsrc, rows_cap, bulk_rows_ok(g, output, VD - 1) ? 1 : 0);
    } else {
        const int rows_cap = rows_cap_for(PD, vd);
        const size_t fixed = sizeof(float) * Cfg<PD>::TP * SliceCfg<PD>::PW + sizeof(int) * Cfg<PD>::TP;
        const size_t smem = sizeof(float) * (size_t)rows_cap * padded_vd(vd) + fixed;
        if (smem > 200 * 1024) return PL_UNSUPPORTED_DIMS;
        PL_TRY((ensure_dynamic_smem<slice_tiles_generic<PD>>(smem)));
        PL_LAUNCH_AFTER(OV_SLICE, (slice_tiles_generic<PD>), tile_grid(g), Cfg<PD>::TP, smem, st, g, output, hdr, tile_info, rec, rec_w,
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
    uint2* srec = reinterpret_cast<uint2*>(ws + L.srec);
    if (srec_words_of(PD) != Cfg<PD>::SREC) return PL_INTERNAL_ERROR;   // the layout and the kernels agree on the stride
    Key<KW>* list_keys = reinterpret_cast<Key<KW>*>(ws + L.list_keys);
    u32* list_ref = reinterpret_cast<u32*>(ws + L.list_ref);
    u32* vid = reinterpret_cast<u32*>(ws + L.vid);
    Key<KW>* vkeys = reinterpret_cast<Key<KW>*>(ws + L.vkeys);
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

    PL_TRY((ensure_dynamic_smem<build_tiles<PD, float>>(Cfg<PD>::BUILD_SMEM)));
    const int sms = num_sms();
    const int wide = sms * 8;
    int table_log2 = 0;
    while ((1ull << table_log2) < L.table_slots) table_log2++;

    // insert_entries overlaps clear_table only while the table can stay in L2 (64 MB of slots): behind a
    // clear_table that itself overlaps build_tiles it cost calls with large tables 4-25 % (pd 16: 30 -> 37 ms)
    const bool small_table = L.table_slots <= (1ull << 23);
    if (phases & PH_BUILD) {
        // a lattice built to be applied later (no values in this call) also gets its splats sorted
        if (phases & PH_APPLY) {
            PL_LAUNCH((build_tiles<PD, float, false>), tile_grid(g), TP, Cfg<PD>::BUILD_SMEM, st, g, positions, reference, hdr,
                                                                         tile_info, rec, rec_w, srec, list_keys, (u32)L.max_entries);
        } else {
            PL_TRY((ensure_dynamic_smem<build_tiles<PD, float, true>>(Cfg<PD>::BUILD_SMEM)));
            PL_LAUNCH((build_tiles<PD, float, true>), tile_grid(g), TP, Cfg<PD>::BUILD_SMEM, st, g, positions, reference, hdr,
                                                                        tile_info, rec, rec_w, srec, list_keys, (u32)L.max_entries);
        }
        PL_COUNT_LAUNCHES(4);   // build_tiles and the three launches of the index stage below
        if (ev) PL_CUDA(cudaEventRecord(ev[1], st));
        Direct direct;
        bool use_direct = false;
        if constexpr (PD <= MAX_SDIMS) use_direct = make_direct(direct, g, PD, L);
        // a new vertex's neighbour slots and (when this call also applies) its value row are initialised
        // by the launch that creates it
        VertexInit vinit;
        vinit.nbr = nbr;
        vinit.max_entries = L.max_entries;
        vinit.pd = PD;
        vinit.rows = (phases & PH_APPLY) ? (v64 ? static_cast<void*>(v64) : static_cast<void*>(v0)) : nullptr;
        vinit.row_bytes = (u32)padded_vd(vd) * (v64 ? 8u : 4u);
        if constexpr (PD <= MAX_SDIMS) {
            if (use_direct) {
                u32* table32 = reinterpret_cast<u32*>(table);
                PL_LAUNCH_AFTER(OV_CLEAR, (clear_direct), wide, 256, 0, st, hdr, table32, direct.slots);
                PL_LAUNCH_AFTER(small_table ? OV_INSERT : 0, (insert_direct<PD>), wide, 256, 0, st, hdr, direct, table32, list_keys, list_ref, vid, vkeys, vinit);
                PL_LAUNCH_AFTER(OV_LINK, (link_neighbours_direct<PD>), wide, 256, 0, st, hdr, direct, table32, list_ref, vid, vkeys, nbr,
                                                                 L.max_entries);
            }
        }
        if (!use_direct) {
            // the value rows are zeroed by the link launch, whose lookups leave the memory system idle
            void* zrows = vinit.rows;
            vinit.rows = nullptr;
            // (behind the build that also sorts the splats the overlap measured slower: 1.66 against 1.61 ms for
            // a build and two applies)
            PL_LAUNCH_AFTER((phases & PH_APPLY) ? OV_CLEAR : 0, (clear_table), wide, 256, 0, st, hdr, table, (u32)table_log2);
            PL_LAUNCH_AFTER(small_table ? OV_INSERT : 0, (insert_entries<KW>), wide, 256, 0, st, hdr, table, list_keys, list_ref, vid, vkeys, vinit);
            PL_LAUNCH_AFTER(OV_LINK, (link_neighbours<PD>), wide, 256, 0, st, hdr, table, list_keys, list_ref, vid, vkeys, nbr,
                                                      L.max_entries, zrows, vinit.row_bytes);
        }
        if (ev) PL_CUDA(cudaEventRecord(ev[2], st));
    } else {
        if (ev) { PL_CUDA(cudaEventRecord(ev[1], st)); }
        PL_LAUNCH((zero_rows), wide, 256, 0, st, hdr, v0, v64, padded_vd(vd));
        PL_COUNT_LAUNCHES(1);
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
        PL_TRY((ensure_dynamic_smem<splat_tiles_det<PD>>(smem)));
        PL_LAUNCH((absmax_kernel), wide, 256, 0, st, input, (u64)g.batch * g.n * (vd - 1), hdr);
        PL_LAUNCH((splat_tiles_det<PD>), tile_grid(g), TP, smem, st, g, input, hdr, tile_info, rec, rec_w, list_ref, v64, vd);
        PL_LAUNCH((convert_fixed), wide, 256, 0, st, hdr, v64, v0, padded_vd(vd));
        PL_COUNT_LAUNCHES(2);   // absmax_kernel, convert_fixed (the splat itself is counted below)
    } else {
        rc = PL_DISPATCH_VD(launch_splat, PD, vd, g, input, hdr, tile_info, rec, rec_w, srec, !(phases & PH_BUILD), list_ref, v0, vd, st);
    }
    if (rc != PL_OK) return rc;
    PL_COUNT_LAUNCHES(1 + 1);   // splat, slice (the blur launches are counted where they are issued)
    if (ev) PL_CUDA(cudaEventRecord(ev[3], st));
    float* src = v0;
    float* dst = v1;
    const int qpr = padded_vd(vd) / 4;
    for (int step = 0; step <= PD; step++) {
        const int axis = reverse ? PD - step : step;
        const int* nb = nbr + (size_t)axis * L.max_entries * 2;
        PL_LAUNCH_AFTER(step == 0 ? OV_BLUR0 : OV_BLUR, (blur_axis), wide, 256, 0, st, hdr, nb, src, dst, qpr);
        float* tmp = src; src = dst; dst = tmp;
    }
    PL_COUNT_LAUNCHES(PD + 1);
    if (ev) PL_CUDA(cudaEventRecord(ev[4], st));
    rc = PL_DISPATCH_VD(launch_slice, PD, vd, g, output, hdr, tile_info, rec, rec_w, list_ref, src, vd, st);
    if (rc != PL_OK) return rc;
    if (ev) PL_CUDA(cudaEventRecord(ev[5], st));
    PL_CUDA(cudaGetLastError());
    return PL_OK;
}

// T = double: the same structure kernels, then splat, blur and slice over rows of doubles.
template <int PD>
static int run_filter_f64(const Geom& g, double* output, const double* input, const double* positions,
                          const double* reference, int vd, int reverse, void* workspace, const Layout& L,
                          cudaStream_t st) {
    constexpr int KW = Cfg<PD>::KW, TP = Cfg<PD>::TP;
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    Header* hdr = reinterpret_cast<Header*>(ws);
    int2* tile_info = reinterpret_cast<int2*>(ws + L.tile_info);
    u16* rec = reinterpret_cast<u16*>(ws + L.rec);
    double* rec_w = reinterpret_cast<double*>(ws + L.rec_w);
    Key<KW>* list_keys = reinterpret_cast<Key<KW>*>(ws + L.list_keys);
    u32* list_ref = reinterpret_cast<u32*>(ws + L.list_ref);
    u32* vid = reinterpret_cast<u32*>(ws + L.vid);
    Key<KW>* vkeys = reinterpret_cast<Key<KW>*>(ws + L.vkeys);
    u64* table = reinterpret_cast<u64*>(ws + L.table);
    int* nbr = reinterpret_cast<int*>(ws + L.nbr);
    double* v0 = reinterpret_cast<double*>(ws + L.v0);
    double* v1 = reinterpret_cast<double*>(ws + L.v1);

    PL_CUDA(cudaMemsetAsync(hdr, 0, sizeof(Header), st));
    if (g.num_tiles == 0) return PL_OK;
    PL_TRY((ensure_dynamic_smem<build_tiles<PD, double>>(Cfg<PD>::BUILD_SMEM)));
    PL_TRY((ensure_dynamic_smem<splat_tiles_f64<PD>>(Splat64<PD>::BYTES)));
    const int wide = num_sms() * 8;
    int table_log2 = 0;
    while ((1ull << table_log2) < L.table_slots) table_log2++;
    const int vp = padded_vd_f64(vd);

    PL_LAUNCH((build_tiles<PD, double>), tile_grid(g), TP, Cfg<PD>::BUILD_SMEM, st, g, positions, reference, hdr, tile_info, rec, rec_w, static_cast<uint2*>(nullptr), list_keys, (u32)L.max_entries);
    // spatial-only calls index their vertices directly, as the float calls do (the key bounds hold for
    // either arithmetic: the margin is far wider than any rounding)
    Direct direct;
    bool use_direct = false;
    if constexpr (PD <= MAX_SDIMS) use_direct = make_direct(direct, g, PD, L);
    u32* table32 = reinterpret_cast<u32*>(table);
    VertexInit vinit;
    vinit.nbr = nbr;
    vinit.max_entries = L.max_entries;
    vinit.pd = PD;
    vinit.rows = v0;   // rows of vp doubles
    vinit.row_bytes = (u32)vp * 8u;
    if constexpr (PD <= MAX_SDIMS) {
        if (use_direct) {
            PL_LAUNCH((clear_direct), wide, 256, 0, st, hdr, table32, direct.slots);
            PL_LAUNCH((insert_direct<PD>), wide, 256, 0, st, hdr, direct, table32, list_keys, list_ref, vid, vkeys, vinit);
            PL_LAUNCH((link_neighbours_direct<PD>), wide, 256, 0, st, hdr, direct, table32, list_ref, vid, vkeys, nbr,
                                                             L.max_entries);
        }
    }
    if (!use_direct) {
        PL_LAUNCH((clear_table), wide, 256, 0, st, hdr, table, (u32)table_log2);
        PL_LAUNCH((insert_entries<KW>), wide, 256, 0, st, hdr, table, list_keys, list_ref, vid, vkeys, vinit);
        PL_LAUNCH((link_neighbours<PD>), wide, 256, 0, st, hdr, table, list_keys, list_ref, vid, vkeys, nbr, L.max_entries,
                                                  nullptr, 0u);
    }
    PL_LAUNCH((splat_tiles_f64<PD>), tile_grid(g), TP, Splat64<PD>::BYTES, st, g, input, hdr, tile_info, rec, rec_w,
                                                                      list_ref, v0, vd);
    double* src = v0;
    double* dst = v1;
    for (int step = 0; step <= PD; step++) {
        const int axis = reverse ? PD - step : step;
        PL_LAUNCH((blur_axis_f64), wide, 256, 0, st, hdr, nbr + (size_t)axis * L.max_entries * 2, src, dst, vp / 2);
        double* tmp = src; src = dst; dst = tmp;
    }
    PL_LAUNCH((slice_tiles_f64<PD>), tile_grid(g), TP, 0, st, g, output, hdr, tile_info, rec, rec_w, list_ref, src, vd);
    PL_COUNT_LAUNCHES(4 + 1 + (PD + 1) + 1);   // build and index (3); splat; blur passes; slice
    PL_CUDA(cudaGetLastError());
    return PL_OK;
}

template <int PD, typename R>
static int run_export(const Geom& g, const R* positions, const R* reference, const void* workspace,
                      const Layout& L, long long max_vertices, int16_t* vertex_keys,
                      int32_t* vertex_item, int32_t* pixel_vertex, R* pixel_weight,
                      cudaStream_t st) {
    constexpr int KW = Cfg<PD>::KW, TP = Cfg<PD>::TP;
    const unsigned char* ws = static_cast<const unsigned char*>(workspace);
    const Header* hdr = reinterpret_cast<const Header*>(ws);
    if (g.num_tiles == 0) return PL_OK;
    if (pixel_vertex || pixel_weight)
        export_points<PD, R><<<tile_grid(g), TP, 0, st>>>(
            g, hdr, reinterpret_cast<const int2*>(ws + L.tile_info), reinterpret_cast<const u16*>(ws + L.rec),
            reinterpret_cast<const R*>(ws + L.rec_w), reinterpret_cast<const u32*>(ws + L.list_ref),
            pixel_vertex, pixel_weight);
    if (vertex_keys || vertex_item)
        export_vertices<PD><<<num_sms() * 4, 256, 0, st>>>(
            hdr, reinterpret_cast<const Key<KW>*>(ws + L.vkeys), max_vertices, vertex_keys, vertex_item);
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
    int rc = make_layout(L, g, pd, vd, max_entries, 4, mode == PL_MODE_DETERMINISTIC);
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
                       int64_t max_entries, int mode, size_t* bytes) {
    if (!bytes || batch < 0 || n < 0 || batch > 65535) return PL_INVALID_ARGUMENT;
    if (mode != PL_MODE_ATOMIC && mode != PL_MODE_DETERMINISTIC) return PL_INVALID_ARGUMENT;
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
    rc = make_layout(L, g, pd, vd, max_entries, 4, mode == PL_MODE_DETERMINISTIC);
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

// ---------------------------------------------------------------------------------------------
// T = double
// ---------------------------------------------------------------------------------------------
static int geom_for_workspace(Geom& g, int batch, int n, int pd, int n_spatial_dims, const int* spatial_dims) {
    if (spatial_dims) {
        if (n_spatial_dims < 1 || n_spatial_dims > MAX_SDIMS || n_spatial_dims > pd) return PL_INVALID_ARGUMENT;
        long long prod = 1;
        for (int i = 0; i < n_spatial_dims; i++) prod *= spatial_dims[i];
        if (prod != n) return PL_INVALID_ARGUMENT;
        return make_geom(g, batch, n, pd, n_spatial_dims, spatial_dims, pd - n_spatial_dims, 1.f, 1.f, false);
    }
    int one = n;
    return make_geom(g, batch, n, pd, 1, &one, pd - 1, 1.f, 1.f, true);
}

int pl_workspace_bytes_f64(int batch, int n, int pd, int vd, int n_spatial_dims, const int* spatial_dims,
                           int64_t max_entries, size_t* bytes) {
    if (!bytes || batch < 0 || n < 0 || batch > 65535) return PL_INVALID_ARGUMENT;
    if (!pl_supported(pd, vd)) return PL_UNSUPPORTED_DIMS;
    Geom g;
    int rc = geom_for_workspace(g, batch, n, pd, n_spatial_dims, spatial_dims);
    if (rc != PL_OK) return rc;
    Layout L;
    rc = make_layout(L, g, pd, vd, max_entries, 8);
    if (rc != PL_OK) return rc;
    *bytes = L.total;
    return PL_OK;
}

int pl_compute_positions_f64(const double* reference, double* positions, int n, int n_reference_channels,
                             int n_spatial_dims, const int* spatial_dims, double spatial_std,
                             double feature_std, void* stream) {
    if (!positions || n < 0 || n_spatial_dims < 0 || n_spatial_dims > MAX_SDIMS ||
        n_reference_channels < 0 || (n_reference_channels > 0 && !reference) ||
        (n_spatial_dims > 0 && !spatial_dims))
        return PL_INVALID_ARGUMENT;
    if (n == 0) return PL_OK;
    Geom g;
    memset(&g, 0, sizeof(g));
    for (int i = 0; i < n_spatial_dims; i++) g.sdims[i] = spatial_dims[i];
    g.spatial_std_d = spatial_std;
    g.feature_std_d = feature_std;
    positions_kernel_f64<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
        reference, positions, n, n_reference_channels, n_spatial_dims, g);
    PL_CUDA(cudaGetLastError());
    return PL_OK;
}

static int filter_common_f64(const Geom& g, double* output, const double* input, const double* positions,
                             const double* reference, int pd, int vd, int reverse, void* workspace,
                             size_t workspace_bytes, int64_t max_entries, cudaStream_t st) {
    Layout L;
    int rc = make_layout(L, g, pd, vd, max_entries, 8);
    if (rc != PL_OK) return rc;
    if (workspace_bytes < L.total) return PL_WORKSPACE_TOO_SMALL;
#define CALL(P) run_filter_f64<P>(g, output, input, positions, reference, vd, reverse, workspace, L, st)
    PL_DISPATCH_PD(pd, CALL)
#undef CALL
}

int pl_filter_f64(double* output, const double* input, const double* positions, int batch, int n, int pd,
                  int vd, int reverse, void* workspace, size_t workspace_bytes, int64_t max_entries,
                  void* stream) {
    if (batch < 0 || n < 0 || batch > 65535) return PL_INVALID_ARGUMENT;
    if (!pl_supported(pd, vd)) return PL_UNSUPPORTED_DIMS;
    if (batch == 0 || n == 0) return PL_OK;
    if (!output || !input || !positions || !workspace) return PL_INVALID_ARGUMENT;
    Geom g;
    int one = n;
    int rc = make_geom(g, batch, n, pd, 1, &one, pd - 1, 1.f, 1.f, true);
    if (rc != PL_OK) return rc;
    set_geom_f64(g, pd, 1.0, 1.0);
    return filter_common_f64(g, output, input, positions, nullptr, pd, vd, reverse, workspace, workspace_bytes,
                             max_entries, (cudaStream_t)stream);
}

int pl_lattice_filter_f64(double* output, const double* input, const double* reference, int batch,
                          int n_spatial_dims, const int* spatial_dims, int n_input_channels,
                          int n_reference_channels, int bilateral, double theta_alpha, double theta_beta,
                          double theta_gamma, int reverse, void* workspace, size_t workspace_bytes,
                          int64_t max_entries, void* stream) {
    if (n_input_channels < 1) return PL_INVALID_ARGUMENT;
    Geom g;
    int pd = 0, n = 0;
    int rc = op_geom(g, batch, n_spatial_dims, spatial_dims, n_reference_channels, bilateral, (float)theta_alpha,
                     (float)theta_beta, (float)theta_gamma, &pd, &n);
    if (rc != PL_OK) return rc;
    set_geom_f64(g, pd, bilateral ? theta_alpha : theta_gamma, bilateral ? theta_beta : -1.0);
    const int vd = n_input_channels + 1;
    if (!pl_supported(pd, vd)) return PL_UNSUPPORTED_DIMS;
    if (batch == 0 || n == 0) return PL_OK;
    if (!output || !input || !workspace || (g.R > 0 && !reference)) return PL_INVALID_ARGUMENT;
    return filter_common_f64(g, output, input, nullptr, reference, pd, vd, reverse, workspace, workspace_bytes,
                             max_entries, (cudaStream_t)stream);
}

int pl_export_lattice_f64(const void* workspace, const double* positions, const double* reference, int batch,
                          int n, int pd, int vd, int n_spatial_dims, const int* spatial_dims,
                          int n_reference_channels, double spatial_std, double feature_std, int64_t max_entries,
                          int64_t max_vertices, int16_t* vertex_keys, int32_t* vertex_item,
                          int32_t* pixel_vertex, double* pixel_weight, void* stream) {
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
        rc = make_geom(g, batch, n, pd, n_spatial_dims, spatial_dims, n_reference_channels, (float)spatial_std,
                       (float)feature_std, false);
    }
    if (rc != PL_OK) return rc;
    set_geom_f64(g, pd, spatial_std, feature_std);
    Layout L;
    rc = make_layout(L, g, pd, vd, max_entries, 8);
    if (rc != PL_OK) return rc;
#define CALL(P) run_export<P, double>(g, positions, reference, workspace, L, (long long)max_vertices, vertex_keys, \
                                      vertex_item, pixel_vertex, pixel_weight, (cudaStream_t)stream)
    PL_DISPATCH_PD(pd, CALL)
#undef CALL
}

#ifdef PL_PHASE_CLOCKS
// Developer aid: resident CTAs per SM of the config-2 tile kernels, as the runtime computes them.
int pl_debug_occupancy(int* out) {
    PL_CUDA(cudaFuncSetAttribute(build_tiles<5>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<5>::BUILD_SMEM));
    PL_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&out[0], build_tiles<5>, 256, Cfg<5>::BUILD_SMEM));
    const size_t ss = SplatRows<5, 22, false>::BYTES;
    PL_CUDA(cudaFuncSetAttribute(splat_tiles_rows<5, 22, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ss));
    PL_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&out[1], splat_tiles_rows<5, 22, false>, 256, ss));
    int rows_cap = (40 * 1024) / (SliceFast<5, 22>::RS * 4);
    const size_t sl = SliceFast<5, 22>::bytes(rows_cap);
    PL_CUDA(cudaFuncSetAttribute(slice_tiles_fast<5, 22>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sl));
    PL_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&out[2], slice_tiles_fast<5, 22>, 256, sl));
    out[3] = (int)Cfg<5>::BUILD_SMEM; out[4] = (int)ss; out[5] = (int)sl;
    cudaFuncAttributes fa;
    PL_CUDA(cudaFuncGetAttributes(&fa, splat_tiles_rows<5, 22, false>));
    out[6] = fa.numRegs; out[7] = (int)fa.sharedSizeBytes;
    return PL_OK;
}

// Developer aid: copies (and clears) the per-kernel phase cycle counters, 8 x 16 values.  SYNCHRONISES.
int pl_debug_phase_cycles(unsigned long long* out) {
    PL_CUDA(cudaDeviceSynchronize());
    PL_CUDA(cudaMemcpyFromSymbol(out, g_phase_cycles, sizeof(unsigned long long) * 8 * 16));
    static unsigned long long zeros[8 * 16] = {0};
    PL_CUDA(cudaMemcpyToSymbol(g_phase_cycles, zeros, sizeof(zeros)));
    return PL_OK;
}
#endif

int pl_crf_update_f32(float* q_out, const float* unaries, const float* q_bilateral, const float* q_spatial,
                      const float* compatibility, float bilateral_weight, float spatial_weight,
                      int64_t n_points, int n_labels, void* stream) {
    if (n_points < 0 || n_labels < 1) return PL_INVALID_ARGUMENT;
    if (n_labels > 128) return PL_UNSUPPORTED_DIMS;
    if (n_points == 0) return PL_OK;
    if (!q_out || !unaries || !q_bilateral || !q_spatial) return PL_INVALID_ARGUMENT;
    cudaStream_t st = (cudaStream_t)stream;
    const int tpb = n_labels <= 32 ? 256 : 128;
    const size_t smem = crf_smem_bytes(tpb, n_labels);
    const long long blocks = (n_points + tpb - 1) / tpb;
    if (blocks > 0x7FFFFFFFll) return PL_INVALID_ARGUMENT;
#define PL_CRF_LAUNCH(TPB, LT)                                                                                   \
    do {                                                                                                         \
        PL_TRY((ensure_dynamic_smem<crf_update<TPB, LT>>(smem)));                                                \
        crf_update<TPB, LT><<<(unsigned)blocks, TPB, smem, st>>>(q_out, unaries, q_bilateral, q_spatial,         \
                                                                 compatibility, bilateral_weight, spatial_weight, \
                                                                 n_points, n_labels);                            \
    } while (0)
    // Potts model at the label count of the benchmark's CRF (20 classes + background): rows in registers
    if (n_labels == 21 && !compatibility) PL_CRF_LAUNCH(256, 21);
    else if (n_labels <= 32) PL_CRF_LAUNCH(256, 0);
    else PL_CRF_LAUNCH(128, 0);
    PL_COUNT_LAUNCHES(1);
#undef PL_CRF_LAUNCH
    PL_CUDA(cudaGetLastError());
    return PL_OK;
}

unsigned long long pl_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int pl_direct_index_min_entries(int batch, int n_spatial_dims, const int* spatial_dims, float theta_gamma,
                                int64_t* min_entries) {
    if (!min_entries || !spatial_dims || batch < 0 || n_spatial_dims < 1) return PL_INVALID_ARGUMENT;
    *min_entries = 0;
    if (n_spatial_dims > MAX_SDIMS || !pd_supported(n_spatial_dims) || batch == 0) return PL_OK;
    float scale[MAX_PD];
    scale_factors(n_spatial_dims, scale);
    Direct d;
    if (!direct_bounds(d, n_spatial_dims, spatial_dims, theta_gamma, scale, batch, ~0ull)) return PL_OK;
    // the index uses the hash table's region as 32-bit slots: 2 * table slots, table slots >= 2 * max_entries
    *min_entries = (int64_t)((d.slots + 3) / 4);
    return PL_OK;
}

int pl_debug_direct_index(int enable) {
    const int was = g_direct_index_enabled;
    g_direct_index_enabled = enable ? 1 : 0;
    return was;
}

int pl_profile_next_call(void** stage_events) {
    g_stage_events = reinterpret_cast<cudaEvent_t*>(stage_events);
    return PL_OK;
}

int pl_lattice_stats(const void* workspace, pl_stats* stats, void* stream) {
    if (!stats) return PL_INVALID_ARGUMENT;
    if (!workspace) {   // the built-in scratch of pl_lattice_filter_f32_noalloc on the current device
        void* scratch = nullptr;
        const int rc = static_scratch_of_current_device(&scratch);
        if (rc != PL_OK) return rc;
        workspace = scratch;
    }
    Header h;
    PL_CUDA(cudaMemcpyAsync(&h, workspace, sizeof(Header), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    PL_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    stats->num_vertices = h.num_vertices;
    stats->num_entries = h.num_entries;
    stats->table_slots = (int64_t)1 << h.table_log2;
    stats->device_status = PL_OK;
    for (int code = PL_INVALID_ARGUMENT; code <= PL_INTERNAL_ERROR; code++)
        if (h.status & (1u << code)) stats->device_status = code;
    stats->direct_index = (int32_t)h.direct;
    stats->max_entries = (int64_t)h.capacity;
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
#define CALL(P) run_export<P, float>(g, positions, reference, workspace, L, (long long)max_vertices, vertex_keys, \
                                     vertex_item, pixel_vertex, pixel_weight, (cudaStream_t)stream)
    PL_DISPATCH_PD(pd, CALL)
#undef CALL
}

}  // extern "C"
