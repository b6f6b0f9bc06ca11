// Blur passes over the vertex rows and the slice stage (interpolate, normalise, write out).
#pragma once
#include "common.cuh"

namespace pl {

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
    // Passes after the first overlap the tail of the pass before (see after_previous_kernel).  The vertex count
    // and the neighbour table are older than any blur pass: a thread's first pair of neighbours is fetched
    // before the wait, so that one of the two dependent loads of its first row is off the critical path.
    const u32 M = hdr->num_vertices;
    const u64 items = (u64)M * qpr;
    const int2* __restrict__ nb = reinterpret_cast<const int2*>(nbr_axis);
    u64 e = (u64)blockIdx.x * blockDim.x + threadIdx.x;
    u32 v = (u32)(e / qpr);
    int2 n = (e < items) ? __ldg(nb + v) : make_int2(-1, -1);
    after_previous_kernel();
    if (hdr->status != 0) return;
    const float4* __restrict__ s = reinterpret_cast<const float4*>(src);
    float4* __restrict__ d = reinterpret_cast<float4*>(dst);
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    while (e < items) {
        const int j = (int)(e - (u64)v * qpr);
        const float4 b = s[e];
        const float4 a = (n.x >= 0) ? s[(u64)n.x * qpr + j] : zero;
        const float4 c = (n.y >= 0) ? s[(u64)n.y * qpr + j] : zero;
        d[e] = make_float4(mix3(a.x, b.x, c.x), mix3(a.y, b.y, c.y), mix3(a.z, b.z, c.z),
                           mix3(a.w, b.w, c.w));
        e += (u64)gridDim.x * blockDim.x;
        if (e < items) {
            v = (u32)(e / qpr);
            n = __ldg(nb + v);
        }
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
    // Launched to overlap the tail of the last blur pass: the status word, the tile's range and the per-point
    // records are older than any blur pass and are fetched before the wait; the vertex rows after it.
    constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS, C = VD - 1, VP = (VD + 3) & ~3, QPR = VP / 4;
    constexpr int RS = SliceFast<PD, VD>::RS;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* rows_s = reinterpret_cast<float*>(smem_raw);                                         // [rows_cap][RS]
    float* out_s = reinterpret_cast<float*>(smem_raw);                                          // [TP][C], later
    int* prow_s = reinterpret_cast<int*>(smem_raw + SliceFast<PD, VD>::region(rows_cap));       // [TP]
    if (call_failed(hdr)) {
        poison_tile_output(g, output, C);
        wait_for_previous_kernel();
        return;
    }
    PhaseClock pc(2);
    const TilePos tpos = this_tile(g);
    const int tid = threadIdx.x, tile = tpos.tile;
    const int2 info = tile_info[tile];
    const int base = info.x, cnt = info.y;
    const int nrows = min(cnt, rows_cap);
    const float4* v4 = reinterpret_cast<const float4*>(vsrc);
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
    wait_for_previous_kernel();
    // Row staging, CH copies per thread and trip: first the vertex numbers of all CH rows (independent
    // loads, in flight together with the record loads above), then the asynchronous copies that depend on
    // them; interleaving them one by one would put a full memory latency between consecutive copies.
    {
        constexpr int CH = 8;
        const int total = nrows * QPR;
        for (int i0 = tid; i0 < total; i0 += CH * TP) {
            u32 vtx[CH];
#pragma unroll
            for (int c = 0; c < CH; c++) {
                const int i = i0 + c * TP;
                vtx[c] = (i < total) ? list_ref[base + i / QPR] : 0u;
            }
#pragma unroll
            for (int c = 0; c < CH; c++) {
                const int i = i0 + c * TP;
                if (i < total) {
                    const int lrow = i / QPR, q = i - lrow * QPR;
                    cp_async16(rows_s + lrow * RS + 4 * q, v4 + (size_t)vtx[c] * QPR + q);
                }
            }
        }
    }
    cp_async_wait_all();
    __syncthreads();
    pc.mark();
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
    pc.mark();
    if (valid) {
        const float inv = (float)(1.0 / (double)acc[C]);
#pragma unroll
        for (int j = 0; j < C; j++) out_s[tid * C + j] = PL_FMUL(acc[j], inv);
    }
    if (bulk_ok) {
        fence_async_proxy();
        __syncthreads();
        pc.mark();
        if (tid < g.TY) {
            int first, count;
            if (tile_row(g, this_tile(g), tid, first, count))   // recomputed: keeps registers free above
                bulk_store(output + (size_t)first * C, out_s + (size_t)tid * g.TX * C, (unsigned)count * C * 4u);
            bulk_store_finish();
        }
        pc.mark();
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
    wait_for_previous_kernel();
    constexpr int TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS, PW = SliceCfg<PD>::PW;
    const int C = vd - 1, VP = padded_vd(vd), QPR = VP >> 2;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float4* rows4 = reinterpret_cast<float4*>(smem_raw);                            // [rows_cap][QPR]
    float* prec_s = reinterpret_cast<float*>(rows4 + (size_t)rows_cap * QPR);       // [TP][PW]
    int* prow_s = reinterpret_cast<int*>(prec_s + (size_t)TP * PW);                 // [TP]
    if (call_failed(hdr)) {
        poison_tile_output(g, output, C);
        return;
    }
    const TilePos tpos = this_tile(g);
    const int tid = threadIdx.x, tile = tpos.tile, lane = tid & 31, warp = tid >> 5;
    const int2 info = tile_info[tile];
    const int base = info.x, cnt = info.y;
    const int nrows = min(cnt, rows_cap);
    const float4* v4 = reinterpret_cast<const float4*>(vsrc);
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
    {   // row staging: vertex numbers of CH rows first, then the copies that depend on them (see slice_tiles_fast)
        constexpr int CH = 8;
        const int total = nrows * QPR;
        for (int i0 = tid; i0 < total; i0 += CH * TP) {
            u32 vtx[CH];
#pragma unroll
            for (int c = 0; c < CH; c++) {
                const int i = i0 + c * TP;
                vtx[c] = (i < total) ? list_ref[base + i / QPR] : 0u;
            }
#pragma unroll
            for (int c = 0; c < CH; c++) {
                const int i = i0 + c * TP;
                if (i < total) cp_async16(rows4 + i, v4 + (size_t)vtx[c] * QPR + (i - (i / QPR) * QPR));
            }
        }
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

}  // namespace pl
