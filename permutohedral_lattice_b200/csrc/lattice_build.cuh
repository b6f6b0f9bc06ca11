// Lattice construction: per-tile key generation and de-duplication (build_tiles), the global hash
// table (clear_table, insert_entries) and the vertex / neighbour tables (insert_entries, link_neighbours).
#pragma once
#include <type_traits>
#include "common.cuh"

namespace pl {

// ---------------------------------------------------------------------------------------------
// build_tiles
// ---------------------------------------------------------------------------------------------
// R: number type of the call (float or double); it decides the geometry arithmetic and the type of the
// stored weights, nothing else.
template <typename R>
struct is_double { static constexpr bool value = false; };
template <>
struct is_double<double> { static constexpr bool value = true; };

// Up to pd = 5 six CTAs fit an SM's shared memory; capping the registers for that (40 per thread, a
// few bytes of spills at pd = 5) measured 13 % faster than five CTAs with 48.
// SORTED (float calls that build a lattice for reuse): also leave every tile's splats sorted by entry in
// `srec`, in the form the splat kernels walk, so that no later splat through this lattice sorts again.
// It costs this kernel a quarter more time and saves every splat a fifth: worth it from the second
// splat on, which is why the one-call filter does not ask for it.
template <int PD, typename R = float, bool SORTED = false>
__global__ void __launch_bounds__(Cfg<PD>::TP, (PD <= 5 && !is_double<R>::value) ? 6 : 1)
build_tiles(Geom g, const R* __restrict__ positions, const R* __restrict__ reference,
            Header* hdr, int2* __restrict__ tile_info, u16* __restrict__ rec, R* __restrict__ rec_w,
            uint2* __restrict__ srec, Key<Cfg<PD>::KW>* __restrict__ list_keys, u32 max_entries) {
    wait_for_previous_kernel();
    constexpr int KW = Cfg<PD>::KW, TP = Cfg<PD>::TP, SPLATS = Cfg<PD>::SPLATS, LS = Cfg<PD>::LS;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Key<KW>* keys_s = reinterpret_cast<Key<KW>*>(smem_raw);
    int* hslots = reinterpret_cast<int*>(smem_raw + Cfg<PD>::BUILD_KEYS);
    u16* lidx_s = reinterpret_cast<u16*>(smem_raw + Cfg<PD>::BUILD_KEYS + sizeof(int) * LS);
    __shared__ int cnt_s[PD + 1], base_s;   // entries per remainder; first global entry of the tile
    __shared__ int wsum_s[TP / 32];

    PhaseClock pc(0);
    const TilePos tpos = this_tile(g);
    const int tid = threadIdx.x, tile = tpos.tile;
    for (int i = tid; i < LS; i += TP) hslots[i] = -1;
    if (tid <= PD) cnt_s[tid] = 0;
    if (tile == 0 && tid == 0) {
        hdr->capacity = max_entries;
        hdr->sorted = SORTED ? 1u : 0u;
    }

    int item, pix, po, py, px;
    const bool valid = tile_point(g, tpos, tid, item, pix, po, py, px);
    u32 slot[PD + 1];   // home slot of each key in the tile's hash, computed while the key is in registers
#pragma unroll
    for (int r = 0; r <= PD; r++) slot[r] = 0;
    if (valid) {
        R f[PD];
        R w[PD + 1];
        load_features<PD>(g, positions, reference, item, pix, po, py, px, f);
        typename std::conditional<is_double<R>::value, Simplex64<PD>, Simplex<PD>>::type s;
        if constexpr (is_double<R>::value) {
            find_simplex_f64<PD>(f, g.scale_d, s);
            barycentric_f64<PD>(s, w);
        } else {
            find_simplex<PD>(f, g.scale, s);
            barycentric<PD>(s, w);
        }
        // the weights are final: store them now so the writes overlap the de-duplication below
        R* recw_tile = rec_w + (size_t)tile * SPLATS;
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
        slot[0] = tile_hash<KW>(k) & (LS - 1);
#pragma unroll
        for (int r = 1; r <= PD; r++) {
#pragma unroll
            for (int i = 0; i < PD; i++)
                k.w[i >> 2] -= (s.rank[i] == PD - r + 1) ? ((u64)(PD + 1) << (16 * (i & 3))) : 0ull;
#pragma unroll
            for (int j = 0; j < KW; j++) k.w[j] += coord_ones<PD>(j);
            keys_s[r * TP + tid] = k;
            slot[r] = tile_hash<KW>(k) & (LS - 1);
        }
    }
    __syncthreads();
    pc.mark();

    // de-duplicate: the first splat to claim a slot for a key represents it.  The first probes of all
    // PD+1 keys are issued together (independent shared-memory accesses); most keys resolve there,
    // the rest walk on one at a time.
    int rep[PD + 1];
    {
        int cand[PD + 1];
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            rep[r] = -1;
            cand[r] = valid ? hslots[slot[r]] : -1;
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
    pc.mark();
    // Number the tile's entries remainder by remainder (all entries of remainder 0 first, ...: the splat
    // stage, which walks the tile's splats in entry order, measured 4 % faster with this order than with
    // entries grouped by warp).  Per warp ONE shared-memory atomic instruction: lane r adds the warp's
    // number of new remainder-r entries to counter r.  The index stored now is relative to the
    // remainder's segment; the segment starts are known after the barrier.
    int* run_s = hslots;   // the tile hash is dead from here on: its memory counts the splats of every entry
    if constexpr (SORTED)
        for (int i = tid; i < SPLATS; i += TP) run_s[i] = 0;
    {
        const int lane = tid & 31;
        unsigned owners[PD + 1];
        int mine = 0;
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            owners[r] = __ballot_sync(0xFFFFFFFFu, valid && rep[r] == r * TP + tid);
            mine = (lane == r) ? __popc(owners[r]) : mine;
        }
        int first = 0;
        if (lane <= PD && mine) first = atomicAdd(&cnt_s[lane], mine);
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            const int first_r = __shfl_sync(0xFFFFFFFFu, first, r);
            if ((owners[r] >> lane) & 1u)
                lidx_s[r * TP + tid] = (u16)(first_r + __popc(owners[r] & ((1u << lane) - 1u)));
        }
    }
    __syncthreads();
    int seg[PD + 1];   // first entry of each remainder's segment
    int cnt = 0;
#pragma unroll
    for (int r = 0; r <= PD; r++) {
        seg[r] = cnt;
        cnt += cnt_s[r];
    }
    if (tid == 0) {
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
    // the per-splat records do not need the tile's first global entry: they are written while thread
    // 0's atomic is in flight
    u16 lfin[PD + 1];
    u16* rec_tile = rec + (size_t)tile * SPLATS;
#pragma unroll
    for (int r = 0; r <= PD; r++) {
        lfin[r] = (valid && rep[r] >= 0) ? (u16)(seg[r] + lidx_s[rep[r]]) : (u16)0;   // the representative has the same remainder
        rec_tile[r * TP + tid] = lfin[r];
    }
    // The tile's splats sorted by entry (what the splat stage walks): a counting sort whose first half,
    // one shared-memory atomic per splat, returns the splat's place inside its entry's run.
    int place[PD + 1];
    if constexpr (SORTED) {
#pragma unroll
        for (int r = 0; r <= PD; r++) place[r] = valid ? atomicAdd(&run_s[lfin[r]], 1) : 0;
    }
    __syncthreads();
    pc.mark();
    if constexpr (!SORTED) let_next_kernel_start();   // what is left of this tile: its keys
    const int base = base_s;
    if (valid && base >= 0) {
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            const int me = r * TP + tid;
            if (rep[r] == me) list_keys[(size_t)base + lfin[r]] = keys_s[me];
        }
    }
    if constexpr (SORTED && !is_double<R>::value) {
        // run starts: exclusive prefix sum of the entries' splat counts (thread t owns entries
        // t (PD+1) .. t (PD+1) + PD)
        const int lane = tid & 31, warp = tid >> 5;
        int local[PD + 1];
        int sum = 0;
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            const int i = tid * (PD + 1) + r;
            local[r] = sum;
            sum += (i < cnt) ? run_s[i] : 0;
        }
        int incl = sum;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int t = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if (lane >= d) incl += t;
        }
        if (lane == 31) wsum_s[warp] = incl;
        __syncthreads();
        int before = 0;
#pragma unroll
        for (int q = 0; q < TP / 32; q++) before += (q < warp) ? wsum_s[q] : 0;
        const int excl = incl - sum + before;
#pragma unroll
        for (int r = 0; r <= PD; r++) {
            const int i = tid * (PD + 1) + r;
            if (i < cnt) run_s[i] = excl + local[r];
        }
        __syncthreads();
        // the list is assembled in shared memory (the key list is dead: the barriers above are behind every
        // thread's key stores) and leaves as one bulk copy
        uint2* sorted_s = reinterpret_cast<uint2*>(smem_raw);
        if (valid) {
            const R* recw_mine = rec_w + (size_t)tile * SPLATS + tid;   // this thread's own earlier stores
#pragma unroll
            for (int r = 0; r <= PD; r++) {
                const int pos = run_s[lfin[r]] + place[r];
                sorted_s[Cfg<PD>::srec_slot(pos)] =
                    make_uint2((unsigned)tid | ((unsigned)lfin[r] << 16), __float_as_uint(recw_mine[r * TP]));
            }
        }
        fence_async_proxy();
        __syncthreads();
        if (tid == 0) {
            bulk_store(srec + (size_t)tile * Cfg<PD>::SREC, sorted_s, (unsigned)(sizeof(uint2) * Cfg<PD>::SREC));
            bulk_store_finish();
        }
    }
    pc.mark(true);
}

// ---------------------------------------------------------------------------------------------
// clear_table: table capacity = power of two >= 2 * entries (at least 1024), chosen on the device.
// ---------------------------------------------------------------------------------------------
__global__ void clear_table(Header* hdr, u64* __restrict__ table, u32 max_log2) {
    after_previous_kernel();
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
// What the insert launch sets up for every vertex it creates, so that no later launch has to: the
// vertex's key (vertex order), its slots of the neighbour table ("missing") and, when `rows` is given,
// its value row (zero).
struct VertexInit {
    int* nbr;            // [pd + 1][max_entries] pairs
    u64 max_entries;
    int pd;
    void* rows;          // value rows to zero (float rows, or the 64-bit sums of the deterministic mode); may be null
    u32 row_bytes;       // bytes of one such row (a multiple of 16)
};

// Entries are inserted in rounds of INSERT_CHUNKS chunks of 256: the winners of a round (entries that
// created a vertex) are collected in shared memory and numbered with ONE atomic on the global vertex
// counter.  One atomic per chunk, all on the same address, was what bounded this launch.
constexpr int INSERT_CHUNKS = 8;
constexpr u32 VERTEX_FLAG = 0x80000000u;   // low word of a table slot: vertex index (set) or entry index (clear)

struct InsertRound {
    u32 t[INSERT_CHUNKS * 256];      // winners of the round: entry ...
    u32 slot[INSERT_CHUNKS * 256];   // ... and the table slot it claimed
    u32 count, base;
};

// Appends a winner to the round's list; one shared-memory atomic per warp.
__device__ __forceinline__ void round_add_winner(InsertRound& rd, bool winner, u32 t, u32 slot) {
    const unsigned ballot = __ballot_sync(0xFFFFFFFFu, winner);
    if (!ballot) return;
    const int lane = threadIdx.x & 31, leader = __ffs(ballot) - 1;
    u32 first = 0;
    if (lane == leader) first = atomicAdd(&rd.count, (u32)__popc(ballot));
    first = __shfl_sync(0xFFFFFFFFu, first, leader);
    if (winner) {
        const u32 pos = first + __popc(ballot & ((1u << lane) - 1u));
        rd.t[pos] = t;
        rd.slot[pos] = slot;
    }
}

// Ends a round: numbers its winners (consecutive vertex indices), writes vid and the vertex-ordered keys,
// initialises the new vertices, and re-labels the winners' table slots with the vertex index, so that a
// lookup ends at the slot (tag, vertex) and the vertex's key instead of walking entry -> owner -> vertex.
// `relabel` writes the slot (hash table: 64-bit slots; direct index: 32-bit slots).  Called by all threads.
template <int KW, typename Relabel>
__device__ __forceinline__ void finish_round(Header* hdr, InsertRound& rd, const Key<KW>* __restrict__ list_keys,
                                             u32* __restrict__ vid, Key<KW>* __restrict__ vkeys,
                                             const VertexInit& vi, Relabel relabel) {
    __syncthreads();
    if (threadIdx.x == 0) rd.base = rd.count ? atomicAdd(&hdr->num_vertices, rd.count) : 0u;
    __syncthreads();
    const u32 base = rd.base, tot = rd.count;
    for (u32 i = threadIdx.x; i < tot; i += 256) {
        const u32 t = rd.t[i], v = base + i;
        vid[t] = v;
        vkeys[v] = list_keys[t];
        __threadfence();              // the key is visible before the slot says "vertex v"
        relabel(rd.slot[i], v);
    }
    if (tot) {
        int2* nb = reinterpret_cast<int2*>(vi.nbr);
        for (int a = 0; a <= vi.pd; a++)
            for (u32 i = threadIdx.x; i < tot; i += 256) nb[(u64)a * vi.max_entries + base + i] = make_int2(-1, -1);
        if (vi.rows) {
            uint4* rows = reinterpret_cast<uint4*>(static_cast<unsigned char*>(vi.rows) + (u64)base * vi.row_bytes);
            const u32 quads = tot * (vi.row_bytes / 16);
            for (u32 i = threadIdx.x; i < quads; i += 256) rows[i] = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) rd.count = 0;
    __syncthreads();
}

// Looks key `k` up in the table.  A slot holds (32-bit hash tag, index): the index of the vertex once its
// creator's round has ended (VERTEX_FLAG set; full key in vkeys), before that the index of the entry that
// created it (full key in list_keys, which the previous launch has completely written).  Returns the low
// word of the matching slot, or 0xFFFFFFFF and the first empty slot met in `empty_slot` (~0 if the
// table is full).
template <int KW>
__device__ __forceinline__ u32 table_probe(const u64* __restrict__ table, u64 mask,
                                           const Key<KW>* __restrict__ list_keys,
                                           const Key<KW>* __restrict__ vkeys, const Key<KW>& k, u64 h,
                                           u64& empty_slot) {
    const u32 tag = (u32)(h >> 32);
    u64 s = h & mask;
    for (u64 it = 0; it <= mask; it++) {
        const u64 cur = table[s];
        if (cur == EMPTY_SLOT) {
            empty_slot = s;
            return 0xFFFFFFFFu;
        }
        if ((u32)(cur >> 32) == tag) {
            const u32 low = (u32)cur;
            const Key<KW>& other = (low & VERTEX_FLAG) ? vkeys[low & ~VERTEX_FLAG] : list_keys[low];
            if (key_equal<KW>(other, k)) return low;
        }
        s = (s + 1) & mask;
    }
    empty_slot = ~0ull;
    return 0xFFFFFFFFu;
}

template <int KW>
__global__ void __launch_bounds__(256)
insert_entries(Header* hdr, u64* __restrict__ table, const Key<KW>* __restrict__ list_keys,
               u32* __restrict__ list_ref, u32* __restrict__ vid, Key<KW>* __restrict__ vkeys, VertexInit vi) {
    after_previous_kernel();
    __shared__ InsertRound rd;
    if (threadIdx.x == 0) rd.count = 0;
    if (call_failed(hdr)) return;   // (its barrier also publishes rd.count)
    const u32 T = hdr->num_entries;
    const u64 mask = (1ull << hdr->table_log2) - 1;
    const u32 stride = gridDim.x * 256u;
    for (u32 start = blockIdx.x * 256u; start < T;) {
        for (int c = 0; c < INSERT_CHUNKS && start < T; c++, start += stride) {
            const u32 t = start + threadIdx.x;
            bool winner = false;
            u64 my_slot = 0;
            if (t < T) {
                const Key<KW> k = list_keys[t];
                const u64 h = hash_key<KW>(k);
                const u64 mine = (h & 0xFFFFFFFF00000000ull) | (u64)t;
                u32 ref = 0xFFFFFFFFu;
                // probe; on an empty slot try to claim it, and keep probing from there if another entry was faster
                u64 s = h & mask;
                for (u64 it = 0; it <= mask; it++) {
                    // slots and vertex keys change during this launch: read them from L2, never from an
                    // L1 line that may predate another CTA's write
                    u64 cur = __ldcg(&table[s]);
                    if (cur == EMPTY_SLOT) {
                        cur = atomicCAS(&table[s], EMPTY_SLOT, mine);
                        if (cur == EMPTY_SLOT) { ref = t; winner = true; my_slot = s; break; }
                    }
                    if ((u32)(cur >> 32) == (u32)(h >> 32)) {
                        const u32 low = (u32)cur;
                        const Key<KW> other = (low & VERTEX_FLAG) ? load_key_l2<KW>(&vkeys[low & ~VERTEX_FLAG])
                                                                  : list_keys[low];
                        if (key_equal<KW>(other, k)) { ref = low; break; }
                    }
                    s = (s + 1) & mask;
                }
                if (ref == 0xFFFFFFFFu) {
                    atomicOr(&hdr->status, 1u << PL_INTERNAL_ERROR);
                    ref = t;
                }
                list_ref[t] = ref;   // owning entry, or (VERTEX_FLAG set) the vertex itself
            }
            round_add_winner(rd, winner, t, (u32)my_slot);
        }
        finish_round<KW>(hdr, rd, list_keys, vid, vkeys, vi, [&](u32 slot, u32 v) {
            table[slot] = (__ldcg(&table[slot]) & 0xFFFFFFFF00000000ull) | (u64)(VERTEX_FLAG | v);
        });
    }
}

// entry -> vertex: after the insert launch list_ref[t] names the entry that owns t's key; the link launch
// turns that into the owner's vertex index (first loop of link_neighbours / link_neighbours_direct).
__device__ __forceinline__ void resolve_entries(const Header* hdr, u32* __restrict__ list_ref,
                                                const u32* __restrict__ vid) {
    const u32 T = hdr->num_entries;
    for (u64 t = (u64)blockIdx.x * blockDim.x + threadIdx.x; t < T; t += (u64)gridDim.x * blockDim.x) {
        const u32 ref = list_ref[t];
        list_ref[t] = (ref & VERTEX_FLAG) ? (ref & ~VERTEX_FLAG) : vid[ref];
    }
}

// ---------------------------------------------------------------------------------------------
// link_neighbours: entry -> vertex, then the +-1 neighbours of every vertex along each of the PD+1
// lattice axes.
// ---------------------------------------------------------------------------------------------
// One table lookup per (vertex v, axis a): the neighbour u whose key is v's key with every stored
// coordinate +1, except coordinate a which moves by -PD (along axis PD no stored coordinate is
// special; src/PermutohedralLatticeCPU.h:381-388).  Then u is v's "+" neighbour and v is u's "-"
// neighbour, so the second lookup of the reference is not needed.  Keys are read in vertex order
// (coalesced); every slot carries a vertex index by now, so a lookup is two dependent accesses.
template <int PD>
__global__ void __launch_bounds__(256)
link_neighbours(const Header* hdr, const u64* __restrict__ table,
                const Key<Cfg<PD>::KW>* __restrict__ list_keys, u32* __restrict__ list_ref,
                const u32* __restrict__ vid, const Key<Cfg<PD>::KW>* __restrict__ vkeys, int* __restrict__ nbr,
                u64 max_entries, void* zero_rows_ptr, u32 zero_row_bytes) {
    after_previous_kernel();
    constexpr int KW = Cfg<PD>::KW;
    if (hdr->status != 0) return;
    resolve_entries(hdr, list_ref, vid);
    const u32 M = hdr->num_vertices;
    const u64 mask = (1ull << hdr->table_log2) - 1;
    if (zero_rows_ptr) {   // streaming stores that overlap the latency of the lookups below
        uint4* rows = reinterpret_cast<uint4*>(zero_rows_ptr);
        const u64 quads = (u64)M * (zero_row_bytes / 16);
        for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += (u64)gridDim.x * blockDim.x)
            rows[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    const u64 items = (u64)M * (PD + 1);
    for (u64 e = (u64)blockIdx.x * blockDim.x + threadIdx.x; e < items; e += (u64)gridDim.x * blockDim.x) {
        // axis-major: neighbouring threads take neighbouring vertices of one axis, so their key loads and
        // their own slots of the neighbour table are contiguous (vertex-major, where the threads of a vertex
        // share one key load, measured slower at pd = 5 and at pd = 16)
        const int a = (int)(e / M);
        const u32 v = (u32)(e - (u64)a * M);
        const Key<KW> k = vkeys[v];
        Key<KW> nk;
#pragma unroll
        for (int j = 0; j < KW; j++) nk.w[j] = 0;
#pragma unroll
        for (int i = 0; i < PD; i++) key_set<KW>(nk, i, (u16)(key_get<KW>(k, i) + ((i == a) ? -PD : 1)));
        key_set<KW>(nk, PD, key_get<KW>(k, PD));
        u64 unused;
        const u32 low = table_probe<KW>(table, mask, list_keys, vkeys, nk, hash_key<KW>(nk), unused);
        if (low != 0xFFFFFFFFu) {
            const u32 u = low & ~VERTEX_FLAG;
            nbr[((u64)a * max_entries + v) * 2] = (int)u;
            nbr[((u64)a * max_entries + u) * 2 + 1] = (int)v;
        }
    }
}

}  // namespace pl
