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
    PhaseClock pc(1);
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
    pc.mark();

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
    pc.mark();

    if (bulk_ok) {
        if (!mbar_wait(&bar, 0)) {
            atomicOr(&hdr->status, 1u << PL_INTERNAL_ERROR);
            return;
        }
    } else {
        cp_async_wait_all();
        __syncthreads();
    }
    pc.mark();

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
#ifdef PL_PHASE_CLOCKS
    if (first < total) {
#else
    if (first >= total) return;
#endif
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
#ifdef PL_PHASE_CLOCKS
    }
    pc.mark(true);
#endif
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

}  // namespace pl
