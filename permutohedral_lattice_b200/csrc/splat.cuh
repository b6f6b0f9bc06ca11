// Splat stage: per-tile sort of the splats by entry and segmented reduction into the vertex rows
// (register-resident, generic and deterministic fixed-point forms).
#pragma once
#include "common.cuh"

namespace pl {

// ---------------------------------------------------------------------------------------------
// splat_tiles: V[vertex] += sum over the tile's splats of weight * [input channels, 1].
// The splats of a tile are counting-sorted by entry in shared memory, then every entry's run is
// summed in registers, reading the tile's input rows from shared memory, and leaves the CTA as one
// vector reduction per 16 bytes.  No floating-point atomics in shared memory.
//
// Narrow rows (VD <= 8, splat_tiles_fast): one THREAD sums a window of PD+1 sorted splats with the whole
// row in registers; the input block arrives by bulk asynchronous copies when its rows are 16-byte aligned.
// Wide rows (8 < VD <= 32, splat_tiles_rows): a quarter warp per window, see there.
// Generic form (any vd): a group of lanes per entry, one float4 of channels per lane.
// ---------------------------------------------------------------------------------------------
template <int PD>
struct SplatCommon {
    static constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS, NW = TP / 32;
    // Words of the sorted list when it is cut into windows (one spare word per window, WL >= PD + 1).
    static constexpr int SORTED = SPLATS + TP;

    // WL > 0 stores sorted position pos at slot(pos): the list is cut into windows of WL splats, each
    // followed by one spare word.  Splats of one entry (written together by neighbouring lanes) land in
    // neighbouring words, and lanes that walk neighbouring windows in step read words WL + 1 apart: an
    // odd number of 8-byte words, so neither side collides on shared-memory banks.
    template <int WL>
    __device__ static __forceinline__ int slot(int pos) {
        if constexpr (WL == 0)
            return pos;
        else
            return pos + pos / WL;
    }

    // Counting sort of the tile's splats by entry.  On return (after the trailing barrier) entry e's
    // splats are sorted positions cur_s[e] .. cur_s[e] + count(e), each stored as
    // (point | entry << 16, weight bits); off_s[e], when given, receives the end of the run.
    // cur_s must be zero for e < nloc on entry.  One shared-memory atomic per splat: the value it
    // returns is the splat's offset inside its entry's run, so no second atomic pass is needed once the
    // run starts are known.  (Grouping equal entries of a warp with a match instruction first measured
    // slower than letting the atomics collide.)
    template <int WL>
    __device__ static __forceinline__ void sort_splats(bool valid, const int* l, const float* w, int nloc,
                                                       uint2* sorted_s, int* cur_s, int* off_s, int* wsum_s) {
        const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
        int off[PD + 1];
#pragma unroll
        for (int r = 0; r <= PD; r++) off[r] = valid ? atomicAdd(&cur_s[l[r]], 1) : 0;
        __syncthreads();
        int local[PD + 1], count[PD + 1];
        int sum = 0;
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            const int i = tid * (PD + 1) + r;
            local[r] = sum;
            count[r] = (i < nloc) ? cur_s[i] : 0;
            sum += count[r];
        }
        int incl = sum;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int t = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if (lane >= d) incl += t;
        }
        if (lane == 31) wsum_s[warp] = incl;
        __syncthreads();
        int before = 0;   // entries' splats counted by the warps below this one (NW broadcast reads, no second barrier)
#pragma unroll
        for (int q = 0; q < NW; q++) before += (q < warp) ? wsum_s[q] : 0;
        const int excl = incl - sum + before;
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            const int i = tid * (PD + 1) + r;
            if (i < nloc) {
                cur_s[i] = excl + local[r];
                if (off_s) off_s[i] = excl + local[r] + count[r];
            }
        }
        __syncthreads();
        if (valid) {
#pragma unroll
            for (int r = 0; r <= PD; r++) {
                const int pos = cur_s[l[r]] + off[r];
                sorted_s[slot<WL>(pos)] = make_uint2((unsigned)tid | ((unsigned)l[r] << 16), __float_as_uint(w[r]));
            }
        }
        __syncthreads();
    }
};

// A splat kernel that expects sorted splats met a lattice without them (pl_lattice_apply_f32 on a workspace
// that no pl_lattice_build*_f32 prepared): the call fails, its output is poisoned by the slice stage.
__device__ __forceinline__ bool lattice_is_sorted(Header* hdr) {
    if (hdr->sorted) return true;
    if (threadIdx.x == 0) atomicOr(&hdr->status, 1u << PL_INVALID_ARGUMENT);
    return false;
}

// The tile's splats as build_tiles sorted them (entry order; (point | entry << 16, weight bits) each),
// copied into the windowed shared-memory list.  The caller's next barrier publishes them.
template <int PD, int WL>
__device__ __forceinline__ void load_sorted_splats(const uint2* __restrict__ srec_tile, int total, uint2* sorted_s) {
    constexpr int TP = Cfg<PD>::TP;
    uint2 v[PD + 1];
#pragma unroll
    for (int r = 0; r <= PD; r++) {
        const int pos = r * TP + (int)threadIdx.x;
        v[r] = (pos < total) ? srec_tile[Cfg<PD>::srec_slot(pos)] : make_uint2(0u, 0u);
    }
#pragma unroll
    for (int r = 0; r <= PD; r++) {
        const int pos = r * TP + (int)threadIdx.x;
        if (pos < total) sorted_s[SplatCommon<PD>::template slot<WL>(pos)] = v[r];
    }
}

// PRE: the lattice was built for reuse and holds every tile's splats already sorted (build_tiles with
// SORTED = true); the kernel copies that list instead of sorting the tile's records.
template <int PD, int VD, bool PRE>
struct SplatFast {
    static constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS, C = VD - 1;
    static constexpr size_t IN_BYTES = ((sizeof(float) * TP * C + 15) / 16) * 16;
    static constexpr int SORTED = SplatCommon<PD>::SORTED;
    static constexpr size_t BYTES = IN_BYTES + sizeof(uint2) * SORTED + (PRE ? 1 : 2) * sizeof(int) * SPLATS + sizeof(int) * TP;
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

template <int PD, int VD, bool PRE>
__global__ void __launch_bounds__(Cfg<PD>::TP)
splat_tiles_fast(Geom g, const float* __restrict__ input, Header* hdr, const int2* __restrict__ tile_info,
                 const u16* __restrict__ rec, const float* __restrict__ rec_w, const uint2* __restrict__ srec,
                 const u32* __restrict__ list_ref, float* __restrict__ v0, int bulk_ok) {
    wait_for_previous_kernel();
    constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS, C = VD - 1, VP = (VD + 3) & ~3;
    using SF = SplatFast<PD, VD, PRE>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* in_s = reinterpret_cast<float*>(smem_raw);                                       // [TP][C]
    uint2* sorted_s = reinterpret_cast<uint2*>(smem_raw + SF::IN_BYTES);                    // [SORTED]
    int* prow_s = reinterpret_cast<int*>(sorted_s + SF::SORTED);                            // [TP]
    u32* vid_s = reinterpret_cast<u32*>(prow_s + TP);                                       // [SPLATS] entry -> vertex
    int* cur_s = reinterpret_cast<int*>(vid_s + SPLATS);                                    // [SPLATS], only without PRE
    __shared__ int wsum_s[32];
    __shared__ __align__(8) u64 bar;
    if (call_failed(hdr)) return;
    if (PRE && !lattice_is_sorted(hdr)) return;
    const TilePos tpos = this_tile(g);
    const int tid = threadIdx.x, tile = tpos.tile;
    const int2 info = tile_info[tile];
    const int base = info.x, nloc = info.y;

    int item, pix;
    const bool valid = tile_point(g, tpos, tid, item, pix);
    prow_s[tid] = valid ? item * g.n + pix : -1;
    for (int i = tid; i < nloc; i += TP) {
        if constexpr (!PRE) cur_s[i] = 0;
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

    const int total = nvalid * (PD + 1);
    if constexpr (PRE) {
        load_sorted_splats<PD, PD + 1>(srec + (size_t)tile * Cfg<PD>::SREC, total, sorted_s);
    } else {
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
    }

    if (bulk_ok) {
        // the outcome of the bounded wait is made uniform over the CTA: either every thread goes on or
        // every thread leaves (after one more bounded wait, so that no copy lands in a CTA that is gone)
        if (!__syncthreads_and(mbar_wait(&bar, 0) ? 1 : 0)) {
            if (tid == 0) atomicOr(&hdr->status, 1u << PL_INTERNAL_ERROR);
            mbar_wait(&bar, 0);
            return;
        }
    } else {
        cp_async_wait_all();
        __syncthreads();
    }

    // Every thread sums a window of PD+1 consecutive sorted splats in registers; whenever the entry
    // changes, and at the end of the window, the partial row leaves as vector reductions.
    const int first = tid * (PD + 1);
    if (first >= total) return;
    float acc[VP];
#pragma unroll
    for (int j = 0; j < VP; j++) acc[j] = 0.f;
    // window tid holds sorted positions first .. first + PD in words tid (PD + 2) + i
    const uint2* sp = sorted_s + tid * (PD + 2);
    int cur = (int)(sp[0].x >> 16);
#pragma unroll
    for (int i = 0; i <= PD; i++) {
        if (first + i < total) {
            const uint2 pw = sp[i];
            const int e = (int)(pw.x >> 16);
            if (e != cur) {
                flush_row<VP>(v0 + (size_t)vid_s[cur] * VP, acc);
                cur = e;
            }
            const float wt = __uint_as_float(pw.y);
            const float* x = in_s + (pw.x & 0xFFFFu) * C;
#pragma unroll
            for (int j = 0; j < C; j++) acc[j] = PL_FMA(wt, x[j], acc[j]);
            acc[C] = PL_FADD(acc[C], wt);
        }
    }
    let_next_kernel_start();   // what is left of this thread's work: its last row
    flush_row<VP>(v0 + (size_t)vid_s[cur] * VP, acc);
}

// Wide rows (8 < VD <= 32): a QUARTER WARP per window.  The input block is staged with rows padded to VP
// floats (16-byte aligned), so the 8 lanes of a quarter warp read one point's row as consecutive
// float4 words: a 128-bit shared-memory load is served one quarter warp at a time, so every quarter
// reads its own row without bank conflicts whatever rows the other quarters read.  Lane h keeps
// channels 4h .. 4h+3 of the running sum; the row's channel C is staged as 1 (homogeneous), the padding
// as 0, so the loop has no channel tests.  A flush is one 16-byte vector reduction per lane.
// PRE: the lattice was built for reuse and holds every tile's splats already sorted, in the windowed form
// (build_tiles with SORTED = true); the list then arrives by one bulk copy, the kernel needs no sort, no
// counters, and fits five CTAs on an SM.
template <int PD, int VD, bool PRE>
struct SplatRows {
    static constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS, VP = (VD + 3) & ~3;
    static constexpr int LR = VP / 4;                  // lanes that hold a piece of the row
    static constexpr int WL = Cfg<PD>::WL;             // splats per window: TP / 8 windows
    static constexpr int SORTED = Cfg<PD>::SREC;
    static constexpr size_t BYTES = sizeof(float) * TP * VP + sizeof(uint2) * SORTED + (PRE ? 0 : sizeof(int) * SPLATS) +
                                    sizeof(int) * TP;
};

// Five CTAs per SM (47-48 registers, no spills; with the sort's counters the five CTAs take nearly all of an
// SM's shared memory): 4 % faster than four at 16 items, and 2048 tiles (two items) take three waves, not four.
template <int PD, int VD, bool PRE>
__global__ void __launch_bounds__(Cfg<PD>::TP, 5)
splat_tiles_rows(Geom g, const float* __restrict__ input, Header* hdr, const int2* __restrict__ tile_info,
                 const u16* __restrict__ rec, const float* __restrict__ rec_w, const uint2* __restrict__ srec,
                 const u32* __restrict__ list_ref, float* __restrict__ v0, int bulk_ok) {
    // Launched to overlap the tail of the kernel before it (link_neighbours, or zero_rows in an apply): all
    // that the staging and the sort read (the input, the records and tile ranges of build_tiles, whose
    // failures are final by now) is older than that kernel, so they run before the wait; the window loop,
    // which reads the entries' vertices and adds to the zeroed rows, runs after it.
    using SR = SplatRows<PD, VD, PRE>;
    constexpr int TP = SR::TP, SPLATS = SR::SPLATS, C = VD - 1, VP = SR::VP, LR = SR::LR, WL = SR::WL;
    static_assert(LR <= 8, "a row must fit the 8 lanes of a quarter warp");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* in_s = reinterpret_cast<float*>(smem_raw);                         // [TP][VP]
    uint2* sorted_s = reinterpret_cast<uint2*>(in_s + TP * VP);               // [SORTED]
    int* prow_s = reinterpret_cast<int*>(sorted_s + SR::SORTED);              // [TP]
    int* cur_s = prow_s + TP;                                                 // [SPLATS], only without PRE
    __shared__ int wsum_s[32];
    __shared__ __align__(8) u64 bar;
    if (call_failed(hdr) || (PRE && !lattice_is_sorted(hdr))) {
        wait_for_previous_kernel();
        return;
    }
    PhaseClock pc(1);
    const TilePos tpos = this_tile(g);
    const int tid = threadIdx.x, tile = tpos.tile, lane = tid & 31, warp = tid >> 5;
    const int2 info = tile_info[tile];
    const int base = info.x, nloc = info.y;

    int item, pix;
    const bool valid = tile_point(g, tpos, tid, item, pix);
    prow_s[tid] = valid ? item * g.n + pix : -1;
    // without PRE the splat records are loaded first: they depend on nothing but the tile number, so their
    // latency overlaps that of the tile's entry range above
    float w[PD + 1];
    int l[PD + 1];
    if constexpr (!PRE) {
        const u16* rec_tile = rec + (size_t)tile * SPLATS;
        const float* recw_tile = rec_w + (size_t)tile * SPLATS;
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            l[r] = valid ? rec_tile[r * TP + tid] : 0;
            w[r] = valid ? recw_tile[r * TP + tid] : 0.f;
        }
        for (int i = tid; i < nloc; i += TP) cur_s[i] = 0;
    }
    if ((PRE || bulk_ok) && tid == 0) mbar_init(&bar, 1);
    const int nvalid = __syncthreads_count(valid);
    const int total = nvalid * (PD + 1);
    pc.mark();
    // PRE: the tile's sorted splats arrive by one bulk copy, already in the windowed form the loop below reads
    constexpr unsigned REC_BYTES = PRE ? (unsigned)(sizeof(uint2) * SR::SORTED) : 0u;
    if ((PRE || bulk_ok) && tid == 0) {
        mbar_expect_tx(&bar, REC_BYTES + (bulk_ok ? (unsigned)nvalid * C * 4u : 0u));
        if constexpr (PRE) bulk_load(sorted_s, srec + (size_t)tile * SR::SORTED, REC_BYTES, &bar);
    }

    // Staging.  Bulk form: every tile row's block (TX points x C floats, contiguous in memory) lands
    // by one bulk asynchronous copy at the END of the tile row's padded region; after the sort a warp
    // spreads it out in place to the padded rows (all reads of a tile row, then all writes: the
    // landing zone overlaps the rows it feeds).  Otherwise: 4-byte asynchronous copies straight to
    // the padded positions.
    const int land = g.TX * (VP - C);   // floats between the start of a tile row's region and its landing zone
    if (bulk_ok) {
        if (tid < g.TY) {
            int first, count;
            if (tile_row(g, tpos, tid, first, count))
                bulk_load(in_s + (size_t)tid * g.TX * VP + land, input + (size_t)first * C, (unsigned)count * C * 4u,
                          &bar);
        }
    } else {
        in_s[tid * VP + C] = 1.f;   // homogeneous channel, then padding
#pragma unroll
        for (int j = C + 1; j < VP; j++) in_s[tid * VP + j] = 0.f;
        // element k = tid, tid + TP, ... of the tile's [point][channel] block; (point, channel) advance
        // without a division: TP = DP * C + DJ
        constexpr int DP = TP / C, DJ = TP % C;
        int p = tid / C, j = tid - p * C;
#pragma unroll 3
        for (int it = 0; it < C; it++) {
            const int row = prow_s[p];
            if (row >= 0) cp_async4(in_s + p * VP + j, input + (size_t)row * C + j);
            p += DP;
            j += DJ;
            if (j >= C) {
                j -= C;
                p++;
            }
        }
    }

    if constexpr (!PRE) SplatCommon<PD>::template sort_splats<WL>(valid, l, w, nloc, sorted_s, cur_s, nullptr, wsum_s);
    pc.mark();
    // did this thread see the copies complete within the bounded wait
    const bool arrived = (PRE || bulk_ok) ? mbar_wait(&bar, 0) : true;
    if (bulk_ok) {
        constexpr int MAXE = (16 * C + 31) / 32;   // elements per lane of a tile row (TX <= 16)
        for (int ly = warp; ly < g.TY; ly += TP / 32) {
            // valid points of this tile row: its first point's validity and the row's width
            const int p0 = ly * g.TX;
            const int row0 = prow_s[p0];
            int count = 0;
            if (row0 >= 0) {
                const int x0 = (row0 % g.n) % g.W;
                count = min(g.TX, g.W - x0);
            }
            float* region = in_s + (size_t)p0 * VP;
            const int n = count * C;
            float tmp[MAXE];
            int dst[MAXE];
            int pp = lane / C, jj = lane - pp * C;   // element e = lane + 32 m is channel jj of point pp
#pragma unroll
            for (int m = 0; m < MAXE; m++) {
                const int e = lane + 32 * m;
                tmp[m] = (e < n) ? region[land + e] : 0.f;
                dst[m] = (e < n) ? pp * VP + jj : -1;
                pp += 32 / C;
                jj += 32 % C;
                if (jj >= C) {
                    jj -= C;
                    pp++;
                }
            }
            __syncwarp();
#pragma unroll
            for (int m = 0; m < MAXE; m++)
                if (dst[m] >= 0) region[dst[m]] = tmp[m];
            if (lane < g.TX) {
                region[lane * VP + C] = 1.f;   // homogeneous channel, then padding
#pragma unroll
                for (int j = C + 1; j < VP; j++) region[lane * VP + j] = 0.f;
            }
        }
    } else {
        cp_async_wait_all();
    }
    // this barrier also makes the outcome of the bounded wait uniform over the CTA: either every thread
    // goes on or every thread leaves (after one more bounded wait, so that no copy lands in a CTA that
    // is gone)
    if (!__syncthreads_and(arrived ? 1 : 0)) {
        if (tid == 0) atomicOr(&hdr->status, 1u << PL_INTERNAL_ERROR);
        mbar_wait(&bar, 0);
        wait_for_previous_kernel();
        return;
    }
    pc.mark();
    wait_for_previous_kernel();
    if (call_failed(hdr)) return;   // a failure of the index stage

    const int h = tid & 7, wnd = tid >> 3, first = wnd * WL;
    const bool active = (h < LR) && (first < total);
    if (active) {
        const int count = min(WL, total - first);
        const uint2* sp = sorted_s + wnd * (WL + 1);   // this window's words (see SplatCommon::slot)
        const float4* in4 = reinterpret_cast<const float4*>(in_s) + h;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        int cur = (int)(sp[0].x >> 16);
        u32 vcur = list_ref[base + cur];   // vertex of the running entry, fetched when the run starts
#pragma unroll 4
        for (int i = 0; i < count; i++) {
            const uint2 pw = sp[i];
            const int e = (int)(pw.x >> 16);
            if (e != cur) {
                red_add_v4(v0 + (size_t)vcur * VP + 4 * h, acc);
                acc = make_float4(0.f, 0.f, 0.f, 0.f);
                cur = e;
                vcur = list_ref[base + cur];
            }
            const float wt = __uint_as_float(pw.y);
            const float4 x = in4[(pw.x & 0xFFFFu) * LR];
            acc.x = PL_FMA(wt, x.x, acc.x);
            acc.y = PL_FMA(wt, x.y, acc.y);
            acc.z = PL_FMA(wt, x.z, acc.z);
            acc.w = PL_FMA(wt, x.w, acc.w);
        }
        let_next_kernel_start();   // what is left of this thread's work: its last row
        red_add_v4(v0 + (size_t)vcur * VP + 4 * h, acc);
    }
    pc.mark(true);
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
    wait_for_previous_kernel();
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
        const int beg = cur_s[e], end = off_s[e];
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
    after_previous_kernel();
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
    after_previous_kernel();
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
    after_previous_kernel();
    if (hdr->status != 0) return;
    const double inv = 1.0 / fixed_scale(hdr);
    const u64 cells = (u64)hdr->num_vertices * vp;
    for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i < cells; i += (u64)gridDim.x * blockDim.x)
        v0[i] = (float)PL_DMUL(__ll2double_rn(v64[i]), inv);
}

// Start of an apply on an already built lattice: value rows (or fixed-point sums) back to zero.
__global__ void __launch_bounds__(256)
zero_rows(Header* hdr, float* __restrict__ v0, long long* __restrict__ v64, int vp) {
    after_previous_kernel();
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

}  // namespace pl
