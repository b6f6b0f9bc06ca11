/* Body of the CPU restatement, instantiated by pl_oracle.c once per number type:
 * REAL = float (names plo_*) and REAL = double (names plo_*_f64).  See pl_oracle.c for what it is. */
typedef struct {
    int pd, vd;
    size_t capacity; /* slots, power of two */
    size_t filled;   /* vertices */
    size_t key_cap;  /* vertices the key/value arrays can hold */
    int32_t* entries; /* slot -> vertex id, -1 empty */
    int16_t* keys;    /* [vertex][pd], creation order */
    REAL* values;    /* [vertex][vd] */
} N(Table);

typedef struct {
    int n, pd, vd;
    N(Table) t;
    int32_t* pix_vertex; /* [n][pd+1] */
    REAL* pix_weight;   /* [n][pd+1] */
    REAL scale[64];
} N(Lattice);

/* Placement only; not part of parity (src/PermutohedralLatticeCPU.h:44-51 uses the same form). */
static inline size_t N(key_hash)(const int16_t* key, int pd) {
    uint64_t k = 0;
    for (int i = 0; i < pd; i++) {
        k += (uint64_t)(int64_t)key[i];
        k *= 2531011u;
    }
    k ^= k >> 29;
    return (size_t)k;
}

static void N(table_init)(N(Table)* t, int pd, int vd, size_t expect_vertices) {
    t->pd = pd;
    t->vd = vd;
    t->capacity = (size_t)1 << 15;
    while (t->capacity < 2 * expect_vertices + 2) t->capacity <<= 1;
    t->filled = 0;
    t->key_cap = t->capacity / 2;
    t->entries = (int32_t*)malloc(t->capacity * sizeof(int32_t));
    memset(t->entries, -1, t->capacity * sizeof(int32_t));
    t->keys = (int16_t*)malloc(t->key_cap * pd * sizeof(int16_t));
    t->values = (REAL*)calloc(t->key_cap * vd, sizeof(REAL));
}

static void N(table_free)(N(Table)* t) {
    free(t->entries);
    free(t->keys);
    free(t->values);
}

static void N(table_grow)(N(Table)* t) {
    size_t old_key_cap = t->key_cap;
    t->capacity *= 2;
    t->key_cap = t->capacity / 2;
    t->keys = (int16_t*)realloc(t->keys, t->key_cap * t->pd * sizeof(int16_t));
    t->values = (REAL*)realloc(t->values, t->key_cap * t->vd * sizeof(REAL));
    memset(t->values + old_key_cap * t->vd, 0, (t->key_cap - old_key_cap) * t->vd * sizeof(REAL));
    free(t->entries);
    t->entries = (int32_t*)malloc(t->capacity * sizeof(int32_t));
    memset(t->entries, -1, t->capacity * sizeof(int32_t));
    size_t mask = t->capacity - 1;
    for (size_t v = 0; v < t->filled; v++) {
        size_t h = N(key_hash)(t->keys + v * t->pd, t->pd) & mask;
        while (t->entries[h] != -1) h = (h + 1) & mask;
        t->entries[h] = (int32_t)v;
    }
}

/* Vertex id of `key`; created when absent and create != 0, else -1.
 * Role of HashTableCPU::lookup / lookupOffset (src/PermutohedralLatticeCPU.h:59-91,163-170). */
static inline int32_t N(table_lookup)(N(Table)* t, const int16_t* key, int create) {
    const int pd = t->pd;
    if (create && t->filled + 1 >= t->key_cap) N(table_grow)(t);
    size_t mask = t->capacity - 1;
    size_t h = N(key_hash)(key, pd) & mask;
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

/* src/PermutohedralLatticeCPU.h:194-217 (compute_scale_factor), T = REAL. */
void N(plo_scale_factors)(int pd, REAL* out) {
    REAL inv_std_dev = (REAL)((pd + 1) * sqrt(2.0 / 3));
    for (int i = 0; i < pd; i++)
        out[i] = (REAL)(1.0 / sqrt((double)((i + 1) * (i + 2))) * (double)inv_std_dev);
}

/* src/PermutohedralLatticeCPU.h:452-474 (compute_kernel_cpu). */
void N(plo_compute_positions)(const REAL* reference, REAL* positions, int n, int n_ref_channels,
                           int n_sdims, const int* sdims, REAL spatial_std, REAL feature_std) {
    int pd = n_sdims + n_ref_channels;
    for (int idx = 0; idx < n; idx++) {
        int divisor = 1;
        for (int s = n_sdims - 1; s >= 0; s--) {
            positions[(size_t)pd * idx + s] = (REAL)((idx / divisor) % sdims[s]) / spatial_std;
            divisor *= sdims[s];
        }
        for (int c = 0; c < n_ref_channels; c++)
            positions[(size_t)pd * idx + n_sdims + c] =
                reference[(size_t)idx * n_ref_channels + c] / feature_std;
    }
}

/* Elevate, enclosing simplex and barycentric weights of one position vector:
 * src/PermutohedralLatticeCPU.h:220-286.  rem0 holds integer values as REALs, as there. */
static inline void N(point_simplex)(const N(Lattice)* L, const REAL* position, REAL* rem0,
                                 int16_t* rank, REAL* bary) {
    const int pd = L->pd;
    REAL el[65];
    /* embed_position_vector (:220-231) */
    REAL sm = 0;
    for (int i = pd; i > 0; i--) {
        /* the reference keeps this product in a float whatever T is (:226) */
        float cf = (float)(position[i - 1] * L->scale[i - 1]);
        el[i] = sm - (REAL)((float)i * cf);
        sm += (REAL)cf;
    }
    el[0] = sm;
    /* find_enclosing_simplex (:233-273) */
    const double inv = 1.0 / (pd + 1);
    int16_t sum = 0;
    for (int i = 0; i <= pd; i++) {
        REAL v = (REAL)((double)el[i] * inv);
        REAL up = (REAL)(ceil((double)v) * (pd + 1));
        REAL down = (REAL)(floor((double)v) * (pd + 1));
        if (up - el[i] < el[i] - down)
            rem0[i] = (REAL)(int16_t)up;
        else
            rem0[i] = (REAL)(int16_t)down;
        sum = (int16_t)((REAL)sum + rem0[i]);
    }
    sum = (int16_t)(sum / (pd + 1));
    for (int i = 0; i <= pd; i++) rank[i] = 0;
    for (int i = 0; i < pd; i++) {
        REAL di = el[i] - rem0[i];
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
            rem0[i] += (REAL)(pd + 1);
        } else if (rank[i] > pd) {
            rank[i] = (int16_t)(rank[i] - (pd + 1));
            rem0[i] -= (REAL)(pd + 1);
        }
    }
    /* compute_barycentric_coordinates (:275-286) */
    for (int i = 0; i < pd + 2; i++) bary[i] = 0;
    for (int i = 0; i <= pd; i++) {
        REAL delta = (REAL)((double)(el[i] - rem0[i]) * inv);
        bary[pd - rank[i]] += delta;
        bary[pd - rank[i] + 1] -= delta;
    }
    bary[0] = (REAL)((double)bary[0] + (1.0 + (double)bary[pd + 1]));
}

/* splat_point / splat (:288-326) */
static void N(lattice_splat)(N(Lattice)* L, const REAL* positions, const REAL* values) {
    const int pd = L->pd, vd = L->vd;
    REAL rem0[65], bary[66];
    int16_t rank[65], key[64];
    for (int n = 0; n < L->n; n++) {
        N(point_simplex)(L, positions + (size_t)n * pd, rem0, rank, bary);
        const REAL* value = values + (size_t)n * (vd - 1);
        for (int r = 0; r <= pd; r++) {
            for (int i = 0; i < pd; i++) {
                key[i] = (int16_t)(rem0[i] + (REAL)r);
                if (rank[i] > pd - r) key[i] = (int16_t)(key[i] - (pd + 1));
            }
            int32_t v = N(table_lookup)(&L->t, key, 1);
            REAL* val = L->t.values + (size_t)v * vd;
            for (int i = 0; i < vd - 1; i++) val[i] += bary[r] * value[i];
            val[vd - 1] += bary[r];
            L->pix_vertex[(size_t)n * (pd + 1) + r] = v;
            L->pix_weight[(size_t)n * (pd + 1) + r] = bary[r];
        }
    }
}

/* blur (:362-415) */
static void N(lattice_blur)(N(Lattice)* L, int reverse) {
    const int pd = L->pd, vd = L->vd;
    N(Table)* t = &L->t;
    REAL* new_values = (REAL*)malloc(t->key_cap * vd * sizeof(REAL));
    REAL* zero = (REAL*)calloc(vd, sizeof(REAL));
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
            const REAL* old_val = t->values + i * vd;
            REAL* new_val = new_values + i * vd;
            int32_t v1 = N(table_lookup)(t, n1, 0);
            int32_t v2 = N(table_lookup)(t, n2, 0);
            const REAL* p1 = v1 < 0 ? zero : t->values + (size_t)v1 * vd;
            const REAL* p2 = v2 < 0 ? zero : t->values + (size_t)v2 * vd;
            for (int k = 0; k < vd; k++)
                new_val[k] = (REAL)(0.25 * (double)p1[k] + 0.5 * (double)old_val[k] +
                                     0.25 * (double)p2[k]);
        }
        REAL* tmp = t->values;
        t->values = new_values;
        new_values = tmp;
    }
    free(new_values);
    free(zero);
}

/* slice_point / slice (:333-358) */
static void N(lattice_slice)(const N(Lattice)* L, REAL* out) {
    const int pd = L->pd, vd = L->vd;
    REAL val[1024];
    for (int n = 0; n < L->n; n++) {
        for (int j = 0; j < vd; j++) val[j] = 0;
        for (int i = 0; i <= pd; i++) {
            REAL w = L->pix_weight[(size_t)n * (pd + 1) + i];
            const REAL* row = L->t.values + (size_t)L->pix_vertex[(size_t)n * (pd + 1) + i] * vd;
            for (int j = 0; j < vd; j++) val[j] += w * row[j];
        }
        REAL scale = (REAL)(1.0 / (double)val[vd - 1]);
        for (int j = 0; j < vd - 1; j++) out[(size_t)n * (vd - 1) + j] = val[j] * scale;
    }
}

/* PermutohedralLatticeCPU::filter (:442-446).  Returns a handle for the queries below (free it
 * with N(plo_free)), or NULL for unsupported sizes (pd > 64 or vd > 1024). */
void* N(plo_filter)(REAL* out, const REAL* in, const REAL* positions, int n, int pd, int vd,
                 int reverse) {
    if (pd < 1 || pd > 64 || vd < 1 || vd > 1024 || n < 0) return NULL;
    N(Lattice)* L = (N(Lattice)*)calloc(1, sizeof(N(Lattice)));
    L->n = n;
    L->pd = pd;
    L->vd = vd;
    N(plo_scale_factors)(pd, L->scale);
    N(table_init)(&L->t, pd, vd, 0);
    L->pix_vertex = (int32_t*)malloc(((size_t)n * (pd + 1) + 1) * sizeof(int32_t));
    L->pix_weight = (REAL*)malloc(((size_t)n * (pd + 1) + 1) * sizeof(REAL));
    N(lattice_splat)(L, positions, in);
    N(lattice_blur)(L, reverse);
    N(lattice_slice)(L, out);
    return L;
}

int N(plo_num_vertices)(void* h) { return (int)((N(Lattice)*)h)->t.filled; }

void N(plo_keys)(void* h, int16_t* keys_out) {
    N(Lattice)* L = (N(Lattice)*)h;
    memcpy(keys_out, L->t.keys, L->t.filled * L->pd * sizeof(int16_t));
}

void N(plo_matrix)(void* h, int32_t* vertex_out, REAL* weight_out) {
    N(Lattice)* L = (N(Lattice)*)h;
    size_t cnt = (size_t)L->n * (L->pd + 1);
    memcpy(vertex_out, L->pix_vertex, cnt * sizeof(int32_t));
    memcpy(weight_out, L->pix_weight, cnt * sizeof(REAL));
}

void N(plo_free)(void* h) {
    N(Lattice)* L = (N(Lattice)*)h;
    if (!L) return;
    N(table_free)(&L->t);
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
    REAL spatial_std, feature_std;
    const REAL *in, *ref;
    REAL* out;
    int failed;
} N(BatchJob);

static void* N(batch_worker)(void* arg) {
    N(BatchJob)* j = (N(BatchJob)*)arg;
    int pd = j->n_sdims + j->c_ref, vd = j->c_in + 1;
    REAL* pos = (REAL*)malloc(((size_t)j->n * pd + 1) * sizeof(REAL));
    for (int b = j->tid; b < j->batch; b += j->threads) {
        const REAL* ref_b = j->ref ? j->ref + (size_t)b * j->n * j->c_ref : NULL;
        N(plo_compute_positions)(ref_b, pos, j->n, j->c_ref, j->n_sdims, j->sdims, j->spatial_std,
                              j->feature_std);
        void* h = N(plo_filter)(j->out + (size_t)b * j->n * j->c_in, j->in + (size_t)b * j->n * j->c_in,
                             pos, j->n, pd, vd, j->reverse);
        if (!h) j->failed = 1;
        N(plo_free)(h);
    }
    free(pos);
    return NULL;
}

double N(plo_filter_batch)(REAL* out, const REAL* in, const REAL* reference, int batch, int n,
                        int n_in_channels, int n_ref_channels, int n_sdims, const int* sdims,
                        REAL spatial_std, REAL feature_std, int reverse, int threads) {
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    N(BatchJob) jobs[256];
    pthread_t th[256];
    struct timespec t0, t1;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (int t = 0; t < threads; t++) {
        N(BatchJob) j = {t,     threads,     batch,       n,  n_in_channels, n_ref_channels, n_sdims,
                      reverse, sdims,     spatial_std, feature_std, in, reference, out, 0};
        jobs[t] = j;
        if (t > 0) pthread_create(&th[t], NULL, N(batch_worker), &jobs[t]);
    }
    N(batch_worker)(&jobs[0]);
    int failed = jobs[0].failed;
    for (int t = 1; t < threads; t++) {
        pthread_join(th[t], NULL);
        failed |= jobs[t].failed;
    }
    clock_gettime(CLOCK_MONOTONIC, &t1);
    if (failed) return -1.0;
    return (double)(t1.tv_sec - t0.tv_sec) + 1e-9 * (double)(t1.tv_nsec - t0.tv_nsec);
}
