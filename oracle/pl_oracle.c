/* TEST INFRASTRUCTURE ONLY: the checker for the CUDA path and the timed CPU baseline.
 * Nothing in the product may call into this file.
 *
 * CPU restatement, in plain C, of the reference's fp32 CPU lattice filter
 * (src/PermutohedralLatticeCPU.h of MiguelMonteiro/permutohedral_lattice, T = float), written so
 * that every floating-point operation happens in the same precision and order as in that header
 * compiled with g++ -O2 -ffp-contract=off.  Build this file with -ffp-contract=off too.
 *
 * Parity status: PINNED.  tests/test_oracle_vs_reference.py checks it bit-for-bit (outputs, vertex
 * keys in creation order, per-pixel vertex ids and weights) against the unmodified header
 * (oracle/ref_shim.cpp) wherever the reference tree is present, and tests/test_oracle_golden.py
 * checks it against fixtures under tests/golden/ that were produced by that header.
 *
 * One deliberate difference: the reference's hash table keeps probing from a stale bucket after it
 * grows (src/PermutohedralLatticeCPU.h:59-62,163-165) and so creates duplicate vertices.  The table
 * here rehashes correctly, which equals the reference run with a table large enough never to grow.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

typedef struct {
    int pd, vd;
    size_t capacity; /* slots, power of two */
    size_t filled;   /* vertices */
    size_t key_cap;  /* vertices the key/value arrays can hold */
    int32_t* entries; /* slot -> vertex id, -1 empty */
    int16_t* keys;    /* [vertex][pd], creation order */
    float* values;    /* [vertex][vd] */
} Table;

typedef struct {
    int n, pd, vd;
    Table t;
    int32_t* pix_vertex; /* [n][pd+1] */
    float* pix_weight;   /* [n][pd+1] */
    float scale[64];
} Lattice;

/* Placement only; not part of parity (src/PermutohedralLatticeCPU.h:44-51 uses the same form). */
static inline size_t key_hash(const int16_t* key, int pd) {
    uint64_t k = 0;
    for (int i = 0; i < pd; i++) {
        k += (uint64_t)(int64_t)key[i];
        k *= 2531011u;
    }
    k ^= k >> 29;
    return (size_t)k;
}

static void table_init(Table* t, int pd, int vd, size_t expect_vertices) {
    t->pd = pd;
    t->vd = vd;
    t->capacity = (size_t)1 << 15;
    while (t->capacity < 2 * expect_vertices + 2) t->capacity <<= 1;
    t->filled = 0;
    t->key_cap = t->capacity / 2;
    t->entries = (int32_t*)malloc(t->capacity * sizeof(int32_t));
    memset(t->entries, -1, t->capacity * sizeof(int32_t));
    t->keys = (int16_t*)malloc(t->key_cap * pd * sizeof(int16_t));
    t->values = (float*)calloc(t->key_cap * vd, sizeof(float));
}

static void table_free(Table* t) {
    free(t->entries);
    free(t->keys);
    free(t->values);
}

static void table_grow(Table* t) {
    size_t old_key_cap = t->key_cap;
    t->capacity *= 2;
    t->key_cap = t->capacity / 2;
    t->keys = (int16_t*)realloc(t->keys, t->key_cap * t->pd * sizeof(int16_t));
    t->values = (float*)realloc(t->values, t->key_cap * t->vd * sizeof(float));
    memset(t->values + old_key_cap * t->vd, 0, (t->key_cap - old_key_cap) * t->vd * sizeof(float));
    free(t->entries);
    t->entries = (int32_t*)malloc(t->capacity * sizeof(int32_t));
    memset(t->entries, -1, t->capacity * sizeof(int32_t));
    size_t mask = t->capacity - 1;
    for (size_t v = 0; v < t->filled; v++) {
        size_t h = key_hash(t->keys + v * t->pd, t->pd) & mask;
        while (t->entries[h] != -1) h = (h + 1) & mask;
        t->entries[h] = (int32_t)v;
    }
}

/* Vertex id of `key`; created when absent and create != 0, else -1.
 * Role of HashTableCPU::lookup / lookupOffset (src/PermutohedralLatticeCPU.h:59-91,163-170). */
static inline int32_t table_lookup(Table* t, const int16_t* key, int create) {
    const int pd = t->pd;
    if (create && t->filled + 1 >= t->key_cap) table_grow(t);
    size_t mask = t->capacity - 1;
    size_t h = key_hash(key, pd) & mask;
    for (;;) {
        int32_t e = t->entries[h];
        if (e == -1) {
            if (!create) return -1;
            memcpy(t->keys + t->filled * pd, key, pd * sizeof(int16_t));
            t->entries[h] = (int32_t)t->filled;
            return (int32_t)(t->filled++);
        }
        if (memcmp(t->keys + (size_t)e * pd, key, pd * sizeof(int16_t)) == 0) return e;
        h = (h + 1) & mask;
    }
}

/* src/PermutohedralLatticeCPU.h:194-217 (compute_scale_factor), T = float. */
void plo_scale_factors(int pd, float* out) {
    float inv_std_dev = (float)((pd + 1) * sqrt(2.0 / 3));
    for (int i = 0; i < pd; i++)
        out[i] = (float)(1.0 / sqrt((double)((i + 1) * (i + 2))) * (double)inv_std_dev);
}

/* src/PermutohedralLatticeCPU.h:452-474 (compute_kernel_cpu). */
void plo_compute_positions(const float* reference, float* positions, int n, int n_ref_channels,
                           int n_sdims, const int* sdims, float spatial_std, float feature_std) {
    int pd = n_sdims + n_ref_channels;
    for (int idx = 0; idx < n; idx++) {
        int divisor = 1;
        for (int s = n_sdims - 1; s >= 0; s--) {
            positions[(size_t)pd * idx + s] = (float)((idx / divisor) % sdims[s]) / spatial_std;
            divisor *= sdims[s];
        }
        for (int c = 0; c < n_ref_channels; c++)
            positions[(size_t)pd * idx + n_sdims + c] =
                reference[(size_t)idx * n_ref_channels + c] / feature_std;
    }
}

/* Elevate, enclosing simplex and barycentric weights of one position vector:
 * src/PermutohedralLatticeCPU.h:220-286.  rem0 holds integer values as floats, as there. */
static inline void point_simplex(const Lattice* L, const float* position, float* rem0,
                                 int16_t* rank, float* bary) {
    const int pd = L->pd;
    float el[65];
    /* embed_position_vector (:220-231) */
    float sm = 0;
    for (int i = pd; i > 0; i--) {
        float cf = position[i - 1] * L->scale[i - 1];
        el[i] = sm - (float)i * cf;
        sm += cf;
    }
    el[0] = sm;
    /* find_enclosing_simplex (:233-273) */
    const double inv = 1.0 / (pd + 1);
    int16_t sum = 0;
    for (int i = 0; i <= pd; i++) {
        float v = (float)((double)el[i] * inv);
        float up = (float)(ceil((double)v) * (pd + 1));
        float down = (float)(floor((double)v) * (pd + 1));
        if (up - el[i] < el[i] - down)
            rem0[i] = (float)(int16_t)up;
        else
            rem0[i] = (float)(int16_t)down;
        sum = (int16_t)((float)sum + rem0[i]);
    }
    sum = (int16_t)(sum / (pd + 1));
    for (int i = 0; i <= pd; i++) rank[i] = 0;
    for (int i = 0; i < pd; i++) {
        float di = el[i] - rem0[i];
        for (int j = i + 1; j <= pd; j++) {
            if (di < el[j] - rem0[j])
                rank[i]++;
            else
                rank[j]++;
        }
    }
    for (int i = 0; i <= pd; i++) {
        rank[i] = (int16_t)(rank[i] + sum);
        if (rank[i] < 0) {
            rank[i] = (int16_t)(rank[i] + pd + 1);
            rem0[i] += (float)(pd + 1);
        } else if (rank[i] > pd) {
            rank[i] = (int16_t)(rank[i] - (pd + 1));
            rem0[i] -= (float)(pd + 1);
        }
    }
    /* compute_barycentric_coordinates (:275-286) */
    for (int i = 0; i < pd + 2; i++) bary[i] = 0;
    for (int i = 0; i <= pd; i++) {
        float delta = (float)((double)(el[i] - rem0[i]) * inv);
        bary[pd - rank[i]] += delta;
        bary[pd - rank[i] + 1] -= delta;
    }
    bary[0] = (float)((double)bary[0] + (1.0 + (double)bary[pd + 1]));
}

/* splat_point / splat (:288-326) */
static void lattice_splat(Lattice* L, const float* positions, const float* values) {
    const int pd = L->pd, vd = L->vd;
    float rem0[65], bary[66];
    int16_t rank[65], key[64];
    for (int n = 0; n < L->n; n++) {
        point_simplex(L, positions + (size_t)n * pd, rem0, rank, bary);
        const float* value = values + (size_t)n * (vd - 1);
        for (int r = 0; r <= pd; r++) {
            for (int i = 0; i < pd; i++) {
                key[i] = (int16_t)(rem0[i] + (float)r);
                if (rank[i] > pd - r) key[i] = (int16_t)(key[i] - (pd + 1));
            }
            int32_t v = table_lookup(&L->t, key, 1);
            float* val = L->t.values + (size_t)v * vd;
            for (int i = 0; i < vd - 1; i++) val[i] += bary[r] * value[i];
            val[vd - 1] += bary[r];
            L->pix_vertex[(size_t)n * (pd + 1) + r] = v;
            L->pix_weight[(size_t)n * (pd + 1) + r] = bary[r];
        }
    }
}

/* blur (:362-415) */
static void lattice_blur(Lattice* L, int reverse) {
    const int pd = L->pd, vd = L->vd;
    Table* t = &L->t;
    float* new_values = (float*)malloc(t->key_cap * vd * sizeof(float));
    float* zero = (float*)calloc(vd, sizeof(float));
    int16_t n1[65], n2[65];
    for (int a = reverse ? pd : 0; a >= 0 && a <= pd; reverse ? a-- : a++) {
        for (size_t i = 0; i < t->filled; i++) {
            const int16_t* key = t->keys + i * pd;
            for (int k = 0; k < pd; k++) {
                n1[k] = (int16_t)(key[k] + 1);
                n2[k] = (int16_t)(key[k] - 1);
            }
            if (a < pd) { /* for a == pd the reference writes a slot its hash never reads */
                n1[a] = (int16_t)(key[a] - pd);
                n2[a] = (int16_t)(key[a] + pd);
            }
            const float* old_val = t->values + i * vd;
            float* new_val = new_values + i * vd;
            int32_t v1 = table_lookup(t, n1, 0);
            int32_t v2 = table_lookup(t, n2, 0);
            const float* p1 = v1 < 0 ? zero : t->values + (size_t)v1 * vd;
            const float* p2 = v2 < 0 ? zero : t->values + (size_t)v2 * vd;
            for (int k = 0; k < vd; k++)
                new_val[k] = (float)(0.25 * (double)p1[k] + 0.5 * (double)old_val[k] +
                                     0.25 * (double)p2[k]);
        }
        float* tmp = t->values;
        t->values = new_values;
        new_values = tmp;
    }
    free(new_values);
    free(zero);
}

/* slice_point / slice (:333-358) */
static void lattice_slice(const Lattice* L, float* out) {
    const int pd = L->pd, vd = L->vd;
    float val[1024];
    for (int n = 0; n < L->n; n++) {
        for (int j = 0; j < vd; j++) val[j] = 0;
        for (int i = 0; i <= pd; i++) {
            float w = L->pix_weight[(size_t)n * (pd + 1) + i];
            const float* row = L->t.values + (size_t)L->pix_vertex[(size_t)n * (pd + 1) + i] * vd;
            for (int j = 0; j < vd; j++) val[j] += w * row[j];
        }
        float scale = (float)(1.0 / (double)val[vd - 1]);
        for (int j = 0; j < vd - 1; j++) out[(size_t)n * (vd - 1) + j] = val[j] * scale;
    }
}

/* PermutohedralLatticeCPU::filter (:442-446).  Returns a handle for the queries below (free it
 * with plo_free), or NULL for unsupported sizes (pd > 64 or vd > 1024). */
void* plo_filter(float* out, const float* in, const float* positions, int n, int pd, int vd,
                 int reverse) {
    if (pd < 1 || pd > 64 || vd < 1 || vd > 1024 || n < 0) return NULL;
    Lattice* L = (Lattice*)calloc(1, sizeof(Lattice));
    L->n = n;
    L->pd = pd;
    L->vd = vd;
    plo_scale_factors(pd, L->scale);
    table_init(&L->t, pd, vd, 0);
    L->pix_vertex = (int32_t*)malloc(((size_t)n * (pd + 1) + 1) * sizeof(int32_t));
    L->pix_weight = (float*)malloc(((size_t)n * (pd + 1) + 1) * sizeof(float));
    lattice_splat(L, positions, in);
    lattice_blur(L, reverse);
    lattice_slice(L, out);
    return L;
}

int plo_num_vertices(void* h) { return (int)((Lattice*)h)->t.filled; }

void plo_keys(void* h, int16_t* keys_out) {
    Lattice* L = (Lattice*)h;
    memcpy(keys_out, L->t.keys, L->t.filled * L->pd * sizeof(int16_t));
}

void plo_matrix(void* h, int32_t* vertex_out, float* weight_out) {
    Lattice* L = (Lattice*)h;
    size_t cnt = (size_t)L->n * (L->pd + 1);
    memcpy(vertex_out, L->pix_vertex, cnt * sizeof(int32_t));
    memcpy(weight_out, L->pix_weight, cnt * sizeof(float));
}

void plo_free(void* h) {
    Lattice* L = (Lattice*)h;
    if (!L) return;
    table_free(&L->t);
    free(L->pix_vertex);
    free(L->pix_weight);
    free(L);
}

/* Batched call with the argument meaning of the lattice_filter op: the per-item loop of
 * src/LatticeFilterKernel.cpp:152-179, items dealt round-robin to `threads` pthreads.
 * Returns wall seconds, or -1 on bad sizes. */
typedef struct {
    int tid, threads, batch, n, c_in, c_ref, n_sdims, reverse;
    const int* sdims;
    float spatial_std, feature_std;
    const float *in, *ref;
    float* out;
    int failed;
} BatchJob;

static void* batch_worker(void* arg) {
    BatchJob* j = (BatchJob*)arg;
    int pd = j->n_sdims + j->c_ref, vd = j->c_in + 1;
    float* pos = (float*)malloc(((size_t)j->n * pd + 1) * sizeof(float));
    for (int b = j->tid; b < j->batch; b += j->threads) {
        const float* ref_b = j->ref ? j->ref + (size_t)b * j->n * j->c_ref : NULL;
        plo_compute_positions(ref_b, pos, j->n, j->c_ref, j->n_sdims, j->sdims, j->spatial_std,
                              j->feature_std);
        void* h = plo_filter(j->out + (size_t)b * j->n * j->c_in, j->in + (size_t)b * j->n * j->c_in,
                             pos, j->n, pd, vd, j->reverse);
        if (!h) j->failed = 1;
        plo_free(h);
    }
    free(pos);
    return NULL;
}

double plo_filter_batch(float* out, const float* in, const float* reference, int batch, int n,
                        int n_in_channels, int n_ref_channels, int n_sdims, const int* sdims,
                        float spatial_std, float feature_std, int reverse, int threads) {
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    BatchJob jobs[256];
    pthread_t th[256];
    struct timespec t0, t1;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (int t = 0; t < threads; t++) {
        BatchJob j = {t,     threads,     batch,       n,  n_in_channels, n_ref_channels, n_sdims,
                      reverse, sdims,     spatial_std, feature_std, in, reference, out, 0};
        jobs[t] = j;
        if (t > 0) pthread_create(&th[t], NULL, batch_worker, &jobs[t]);
    }
    batch_worker(&jobs[0]);
    int failed = jobs[0].failed;
    for (int t = 1; t < threads; t++) {
        pthread_join(th[t], NULL);
        failed |= jobs[t].failed;
    }
    clock_gettime(CLOCK_MONOTONIC, &t1);
    if (failed) return -1.0;
    return (double)(t1.tv_sec - t0.tv_sec) + 1e-9 * (double)(t1.tv_nsec - t0.tv_nsec);
}
