/*
 * TEST INFRASTRUCTURE ONLY.
 *
 * CPU restatement (plain C) of the reference algorithms on the sparse-embedding
 * hot path.  It is the checker the parity tests compare the CUDA path against
 * and the "port" CPU baseline timed by the benchmark; nothing in the product
 * path links, loads or calls it.
 *
 * Parity pinning: every function here is checked (tests/test_oracle_*.py)
 * against the reference's own compiled host code (oracle/_ref, built from the
 * reference tree by oracle/build_ref.py), against fixtures generated from it
 * (tests/golden/), against torch.nn.EmbeddingBag + torch.optim -- the golden
 * the reference's operator test uses -- and against the hand examples in the
 * reference's unit tests.
 *
 * All reference citations are paths inside the reference project.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC oracle.c -o liboracle.so -lm
 * (-ffp-contract=off: every float operation is rounded separately, the way
 * the reference's vector instructions Mul/Muls/Add/Div/Sqrt are.)
 */
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_OK 0

/* Threads of the OpenMP loops below, set explicitly by the timing harness (a launcher that exports
 * OMP_NUM_THREADS=1 to its workers must not decide a multi-core baseline).  Returns the count in effect. */
int orc_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}
#define ORC_ERR_NEGATIVE_KEY 1
#define ORC_ERR_TABLE_FULL 2
#define ORC_ERR_CACHE_TOO_SMALL 3
#define ORC_ERR_BAD_ARG 4

/* ------------------------------------------------------------------------- */
/* int64 -> int64 open-addressing map (stands in for ska::flat_hash_map and   */
/* std::unordered_map in the reference; only lookups/inserts/erases, whose    */
/* results do not depend on the container).                                   */
/* ------------------------------------------------------------------------- */
typedef struct {
    int64_t* keys;
    int64_t* vals;
    uint8_t* state; /* 0 empty, 1 full, 2 tombstone */
    uint64_t cap;   /* power of two */
    uint64_t used;  /* full + tombstones */
    uint64_t live;
} orc_map;

static uint64_t orc_mix(uint64_t x)
{
    x ^= x >> 33;
    x *= 0xff51afd7ed558ccdULL;
    x ^= x >> 33;
    x *= 0xc4ceb9fe1a85ec53ULL;
    x ^= x >> 33;
    return x;
}

static void orc_map_init(orc_map* m, uint64_t cap_hint)
{
    uint64_t cap = 16;
    while (cap < cap_hint * 2) cap <<= 1;
    m->cap = cap;
    m->used = 0;
    m->live = 0;
    m->keys = (int64_t*)malloc(cap * sizeof(int64_t));
    m->vals = (int64_t*)malloc(cap * sizeof(int64_t));
    m->state = (uint8_t*)calloc(cap, 1);
}

static void orc_map_free(orc_map* m)
{
    free(m->keys);
    free(m->vals);
    free(m->state);
}

static int64_t* orc_map_find(const orc_map* m, int64_t key)
{
    uint64_t mask = m->cap - 1;
    uint64_t i = orc_mix((uint64_t)key) & mask;
    while (m->state[i] != 0) {
        if (m->state[i] == 1 && m->keys[i] == key) return &m->vals[i];
        i = (i + 1) & mask;
    }
    return NULL;
}

static void orc_map_put(orc_map* m, int64_t key, int64_t val);

static void orc_map_grow(orc_map* m)
{
    orc_map n;
    uint64_t i;
    orc_map_init(&n, m->live * 2 + 8);
    for (i = 0; i < m->cap; i++)
        if (m->state[i] == 1) orc_map_put(&n, m->keys[i], m->vals[i]);
    orc_map_free(m);
    *m = n;
}

static void orc_map_put(orc_map* m, int64_t key, int64_t val)
{
    uint64_t mask, i;
    int64_t* f = orc_map_find(m, key);
    if (f) {
        *f = val;
        return;
    }
    if ((m->used + 1) * 10 > m->cap * 7) orc_map_grow(m);
    mask = m->cap - 1;
    i = orc_mix((uint64_t)key) & mask;
    while (m->state[i] == 1) i = (i + 1) & mask;
    if (m->state[i] == 0) m->used++;
    m->state[i] = 1;
    m->keys[i] = key;
    m->vals[i] = val;
    m->live++;
}

static void orc_map_erase(orc_map* m, int64_t key)
{
    int64_t* f = orc_map_find(m, key);
    if (!f) return;
    m->state[f - m->vals] = 2;
    m->live--;
}

/* ------------------------------------------------------------------------- */
/* A1  sorted unique + inverse                                                */
/* hybrid_torchrec/src/ids_process/unique.cpp:55-117 (UniqueCpuSortedTemplate),*/
/* :120-127 (UniqueParallel): sort, adjacent-diff, inverse[perm[i]] = rank.   */
/* ------------------------------------------------------------------------- */
typedef struct {
    int64_t key;
    int64_t pos;
} orc_pair;

static int orc_pair_cmp(const void* a, const void* b)
{
    const orc_pair* x = (const orc_pair*)a;
    const orc_pair* y = (const orc_pair*)b;
    if (x->key != y->key) return x->key < y->key ? -1 : 1;
    return x->pos < y->pos ? -1 : (x->pos > y->pos);
}

int64_t orc_unique_sorted(const int64_t* ids, int64_t n, int64_t* unique_out, int64_t* inverse_out)
{
    int64_t i, u = 0;
    orc_pair* p;
    if (n == 0) return 0;
    p = (orc_pair*)malloc((size_t)n * sizeof(orc_pair));
    for (i = 0; i < n; i++) {
        p[i].key = ids[i];
        p[i].pos = i;
    }
    qsort(p, (size_t)n, sizeof(orc_pair), orc_pair_cmp);
    for (i = 0; i < n; i++) {
        if (i == 0 || p[i].key != p[i - 1].key) unique_out[u++] = p[i].key;
        inverse_out[p[i].pos] = u - 1;
    }
    free(p);
    return u;
}

/* ------------------------------------------------------------------------- */
/* A2  IdsMapper: key -> slot in first-come order, then first-occurrence      */
/* unique of the slots of one table segment.                                  */
/* hybrid_torchrec/src/ids_process/ids_mapper.cpp:36-61 (FindOrInsert...),    */
/* :63-113 (UniqueAndLookupOut), :115-174 (UniqueProcessing); class state     */
/* ids_mapper.h:91-98 (ids2indicesMap, indice2id, maxIndex, initMaxIndex,     */
/* onlyDeviceMem).                                                            */
/* ------------------------------------------------------------------------- */
typedef struct {
    orc_map map;
    int64_t* slot2id;
    int64_t slot2id_cap;
    int64_t max_index;
    int64_t init_max_index;
    int only_device_mem;
} orc_mapper;

void* orc_mapper_new(int64_t init_max_index, int only_device_mem)
{
    orc_mapper* m = (orc_mapper*)calloc(1, sizeof(orc_mapper));
    orc_map_init(&m->map, 1024);
    m->slot2id_cap = 1024;
    m->slot2id = (int64_t*)malloc((size_t)m->slot2id_cap * sizeof(int64_t));
    m->init_max_index = init_max_index;
    m->only_device_mem = only_device_mem;
    return m;
}

void orc_mapper_free(void* h)
{
    orc_mapper* m = (orc_mapper*)h;
    orc_map_free(&m->map);
    free(m->slot2id);
    free(m);
}

int64_t orc_mapper_size(void* h) { return ((orc_mapper*)h)->max_index; }

static int orc_mapper_find_or_insert(orc_mapper* m, int64_t key, int64_t* slot, int check_full)
{
    int64_t* f;
    if (key < 0) return ORC_ERR_NEGATIVE_KEY; /* ids_mapper.cpp:45,83 */
    f = orc_map_find(&m->map, key);
    if (f) {
        *slot = *f;
        return ORC_OK;
    }
    if (check_full && m->max_index >= m->init_max_index) return ORC_ERR_TABLE_FULL; /* :48-50, :93-97 */
    *slot = m->max_index++;
    orc_map_put(&m->map, key, *slot);
    if (*slot >= m->slot2id_cap) {
        m->slot2id_cap *= 2;
        m->slot2id = (int64_t*)realloc(m->slot2id, (size_t)m->slot2id_cap * sizeof(int64_t));
    }
    m->slot2id[*slot] = key;
    return ORC_OK;
}

/* ids2indices_unique: slots for all ids, then SORTED unique of the slots
 * (ids_mapper.cpp:36-61 -> UniqueParallel).  Returns U or a negative error. */
int64_t orc_mapper_ids2indices_unique(void* h, const int64_t* ids, int64_t n, int64_t* hash_indices,
                                      int64_t* unique_out, int64_t* inverse_out)
{
    orc_mapper* m = (orc_mapper*)h;
    int64_t i;
    for (i = 0; i < n; i++) {
        int rc = orc_mapper_find_or_insert(m, ids[i], &hash_indices[i], 1);
        if (rc != ORC_OK) return -rc;
    }
    return orc_unique_sorted(hash_indices, n, unique_out, inverse_out);
}

/* ids2indices_unique_out for one table (ids_mapper.cpp:63-174).  The segment is
 * [offset[table_id], offset[table_id+1]); unique_offset[table_id] must already
 * hold this table's base (0 for table 0). */
int orc_mapper_unique_out(void* h, const int64_t* ids, int64_t* hash_indices, const int64_t* offset,
                          int64_t* unique, int64_t* unique_ids, int64_t* unique_inverse,
                          int64_t* unique_offset, int64_t table_id)
{
    orc_mapper* m = (orc_mapper*)h;
    int64_t start = offset[table_id], end = offset[table_id + 1];
    int64_t i, base, cnt = 0;
    int64_t* first;
    if (start == end) {
        unique_offset[table_id + 1] = unique_offset[table_id];
        return ORC_OK;
    }
    for (i = start; i < end; i++) {
        int rc = orc_mapper_find_or_insert(m, ids[i], &hash_indices[i], m->only_device_mem);
        if (rc != ORC_OK) return rc;
    }
    base = unique_offset[table_id];
    first = (int64_t*)malloc((size_t)m->max_index * sizeof(int64_t));
    for (i = 0; i < m->max_index; i++) first[i] = -1;
    for (i = start; i < end; i++) { /* :143-151 first occurrence order */
        int64_t s = hash_indices[i];
        if (first[s] == -1) {
            first[s] = cnt;
            unique[base + cnt] = s;
            unique_ids[base + cnt] = m->slot2id[s];
            cnt++;
        }
    }
    if (table_id == 0) unique_offset[0] = 0;
    unique_offset[table_id + 1] = unique_offset[table_id] + cnt;
    for (i = start; i < end; i++) unique_inverse[i] = first[hash_indices[i]]; /* :163-166 */
    free(first);
    return ORC_OK;
}

/* ------------------------------------------------------------------------- */
/* A3  row-hash bucketize                                                     */
/* hybrid_torchrec/src/ids_process/bucketize.cpp:35-51 (ComputeNewLengths),   */
/* :54-76 (FillNewIndices), :79-130 (Deduplicate), :133-211 (driver).         */
/* lengths is [F*B]; bucket = id % W; new layout is bucket-major.             */
/* Returns the number of valid entries in new_indices (N, or the unique count */
/* when do_unique).                                                           */
/* ------------------------------------------------------------------------- */
int64_t orc_bucketize(const int64_t* lengths, int64_t lengths_size, const int64_t* indices, int64_t n,
                      int64_t num_features, int64_t W, int sequence, int do_unique, int return_count,
                      int64_t* new_lengths /* [W*F*B], zeroed here */, int64_t* new_indices /* [N] */,
                      int64_t* unbucketize_permute /* [N] */, int64_t* ids_counts /* [N] or NULL */)
{
    int64_t B = lengths_size / num_features;
    int64_t nl = lengths_size * W;
    int64_t* offs = (int64_t*)malloc((size_t)(lengths_size + 1) * sizeof(int64_t));
    int64_t* noffs = (int64_t*)malloc((size_t)(nl + 1) * sizeof(int64_t));
    int64_t f, b, i, result = n;
    offs[0] = 0;
    for (i = 0; i < lengths_size; i++) offs[i + 1] = offs[i] + lengths[i];
    memset(new_lengths, 0, (size_t)nl * sizeof(int64_t));
    for (f = 0; f < num_features; f++)
        for (b = 0; b < B; b++) {
            int64_t lin = f * B + b;
            for (i = offs[lin]; i < offs[lin + 1]; i++) new_lengths[(indices[i] % W) * lengths_size + lin]++;
        }
    noffs[0] = 0;
    for (i = 0; i < nl; i++) noffs[i + 1] = noffs[i] + new_lengths[i];
    for (f = 0; f < num_features; f++)
        for (b = 0; b < B; b++) {
            int64_t lin = f * B + b;
            for (i = offs[lin]; i < offs[lin + 1]; i++) {
                int64_t bucket = indices[i] % W;
                int64_t pos = noffs[bucket * lengths_size + lin]++;
                new_indices[pos] = indices[i];
                if (sequence) unbucketize_permute[i] = pos;
            }
        }
    /* after the fill, noffs[x] is the END of segment x (bucketize.cpp:70) */
    if (sequence && do_unique) {
        int64_t nmaps = num_features * W, fb, uniq = 0, last = 0;
        orc_map* maps = (orc_map*)malloc((size_t)nmaps * sizeof(orc_map));
        for (fb = 0; fb < nmaps; fb++) orc_map_init(&maps[fb], 16);
        for (fb = 0; fb < nmaps; fb++) {
            for (b = 0; b < B; b++) {
                int64_t lin = fb * B + b;
                int64_t s = last, e = noffs[lin];
                last = e;
                for (i = s; i < e; i++) {
                    int64_t idx = new_indices[i];
                    int64_t* hit = orc_map_find(&maps[fb], idx);
                    if (!hit) {
                        orc_map_put(&maps[fb], idx, uniq);
                        new_indices[uniq] = idx;
                        if (return_count) ids_counts[uniq] = 1;
                        uniq++;
                    } else {
                        if (return_count) ids_counts[*hit]++;
                        new_lengths[lin]--;
                    }
                }
            }
        }
        for (f = 0; f < num_features; f++)
            for (b = 0; b < B; b++) {
                int64_t lin = f * B + b;
                for (i = offs[lin]; i < offs[lin + 1]; i++) {
                    int64_t bucket = indices[i] % W;
                    unbucketize_permute[i] = *orc_map_find(&maps[bucket * num_features + f], indices[i]);
                }
            }
        for (fb = 0; fb < nmaps; fb++) orc_map_free(&maps[fb]);
        free(maps);
        result = uniq;
    }
    free(offs);
    free(noffs);
    return result;
}

/* ------------------------------------------------------------------------- */
/* A4  SwapManager: HBM cache slot policy                                     */
/* torchrec_embcache/csrc/embedding_cache/swap_manager.cpp:20-30 (ctor),      */
/* :32-139 (ComputeSwapInfo), :141-159 (RemoveKeys); state swap_manager.h:41-54*/
/* ------------------------------------------------------------------------- */
typedef struct {
    orc_map key2off;
    int64_t* slot_key;
    int64_t* slot_version;
    int64_t cache_size, mem_start, occupied, now_version, swap_idx;
} orc_swap;

void* orc_swap_new(int64_t cache_size, int64_t mem_start)
{
    orc_swap* s = (orc_swap*)calloc(1, sizeof(orc_swap));
    orc_map_init(&s->key2off, 1024);
    s->slot_key = (int64_t*)calloc((size_t)cache_size, sizeof(int64_t));
    s->slot_version = (int64_t*)calloc((size_t)cache_size, sizeof(int64_t));
    s->cache_size = cache_size;
    s->mem_start = mem_start;
    s->occupied = mem_start;
    s->swap_idx = mem_start;
    return s;
}

void orc_swap_free(void* h)
{
    orc_swap* s = (orc_swap*)h;
    orc_map_free(&s->key2off);
    free(s->slot_key);
    free(s->slot_version);
    free(s);
}

int orc_swap_compute(void* h, const int64_t* keys, int64_t n, int64_t* batch_offs, int64_t* swapin_keys,
                     int64_t* swapin_offs, int64_t* n_swapin, int64_t* swapout_keys, int64_t* swapout_offs,
                     int64_t* n_swapout)
{
    orc_swap* s = (orc_swap*)h;
    int64_t i, nin = 0, nout = 0, nmiss = 0;
    int64_t* missed = (int64_t*)malloc((size_t)(n > 0 ? n : 1) * sizeof(int64_t));
    for (i = 0; i < n; i++) { /* hit pass :45-67 */
        int64_t key = keys[i];
        int64_t* f;
        if (key == -1) {
            batch_offs[i] = 0;
            continue;
        }
        f = orc_map_find(&s->key2off, key);
        if (f) {
            batch_offs[i] = *f;
            s->slot_version[*f] = s->now_version;
        } else {
            missed[nmiss++] = i;
        }
    }
    for (i = 0; i < nmiss; i++) { /* miss loop :81-136, in input order */
        int64_t p = missed[i], key = keys[p], off, old_key;
        int64_t* f = orc_map_find(&s->key2off, key);
        int evicted_pos;
        if (f) {
            batch_offs[p] = *f;
            continue;
        }
        if (s->occupied < s->cache_size) {
            off = s->occupied++;
            swapin_keys[nin] = key;
            swapin_offs[nin++] = off;
            s->slot_key[off] = key;
            s->slot_version[off] = s->now_version;
            orc_map_put(&s->key2off, key, off);
            batch_offs[p] = off;
            continue;
        }
        while (s->swap_idx < s->cache_size && s->slot_version[s->swap_idx] >= s->now_version - 1) s->swap_idx++;
        if (s->swap_idx == s->cache_size) {
            s->swap_idx = s->mem_start;
            while (s->swap_idx < s->cache_size && s->slot_version[s->swap_idx] >= s->now_version - 1) s->swap_idx++;
            if (s->swap_idx == s->cache_size) {
                free(missed);
                return ORC_ERR_CACHE_TOO_SMALL;
            }
        }
        evicted_pos = s->slot_version[s->swap_idx] == -2;
        off = s->swap_idx++;
        swapin_keys[nin] = key;
        swapin_offs[nin++] = off;
        old_key = s->slot_key[off];
        if (old_key != -1) orc_map_erase(&s->key2off, old_key);
        if (!evicted_pos) {
            swapout_keys[nout] = old_key;
            swapout_offs[nout++] = off;
        }
        s->slot_key[off] = key;
        s->slot_version[off] = s->now_version;
        orc_map_put(&s->key2off, key, off);
        batch_offs[p] = off;
    }
    s->now_version++;
    *n_swapin = nin;
    *n_swapout = nout;
    free(missed);
    return ORC_OK;
}

void orc_swap_remove(void* h, const int64_t* keys, int64_t n)
{
    orc_swap* s = (orc_swap*)h;
    int64_t i;
    for (i = 0; i < n; i++) {
        int64_t* f = orc_map_find(&s->key2off, keys[i]);
        if (!f) continue;
        s->slot_version[*f] = -2;
        s->slot_key[*f] = -1;
        orc_map_erase(&s->key2off, keys[i]);
    }
}

int64_t orc_swap_occupied(void* h) { return ((orc_swap*)h)->occupied; }

/* ------------------------------------------------------------------------- */
/* A5  FeatureFilter: count-based admission and timestamp eviction            */
/* torchrec_embcache/csrc/feature_filter/feature_filter.cpp:112-138           */
/* (StatisticsKeyCount), :140-160 (CountFilter), :27-50 (RecordTimestamp),    */
/* :52-80 (FeatureEvict).  The order of the evicted keys in the reference is  */
/* the iteration order of a std::unordered_map, i.e. unspecified; here they   */
/* are reported in ascending key order and compared as a set.                 */
/* ------------------------------------------------------------------------- */
typedef struct {
    orc_map count;
    orc_map ts;
    int64_t admit_threshold; /* -1 = disabled */
    uint64_t evict_threshold, evict_interval, record_batch_id;
    int64_t latest_ts;
    int64_t* evict_keys;
    int64_t n_evict, evict_cap;
} orc_filter;

void* orc_filter_new(int64_t admit_threshold, uint64_t evict_threshold, uint64_t evict_interval)
{
    orc_filter* f = (orc_filter*)calloc(1, sizeof(orc_filter));
    orc_map_init(&f->count, 1024);
    orc_map_init(&f->ts, 1024);
    f->admit_threshold = admit_threshold;
    f->evict_threshold = evict_threshold;
    f->evict_interval = evict_interval;
    f->evict_cap = 1024;
    f->evict_keys = (int64_t*)malloc((size_t)f->evict_cap * sizeof(int64_t));
    return f;
}

void orc_filter_free(void* h)
{
    orc_filter* f = (orc_filter*)h;
    orc_map_free(&f->count);
    orc_map_free(&f->ts);
    free(f->evict_keys);
    free(f);
}

void orc_filter_statistics(void* h, const int64_t* keys, const int64_t* counts, int64_t n)
{
    orc_filter* f = (orc_filter*)h;
    int64_t i;
    for (i = 0; i < n; i++) {
        int64_t c = counts ? counts[i] : 1;
        int64_t* hit;
        if (c < 0) c = 0;
        hit = orc_map_find(&f->count, keys[i]);
        if (hit)
            *hit += c;
        else
            orc_map_put(&f->count, keys[i], c);
    }
}

void orc_filter_count_filter(void* h, int64_t* keys, int64_t n)
{
    orc_filter* f = (orc_filter*)h;
    int64_t i;
    if (f->admit_threshold == -1) return;
    for (i = 0; i < n; i++) {
        int64_t* hit = orc_map_find(&f->count, keys[i]);
        if (hit && (uint64_t)*hit < (uint64_t)f->admit_threshold) keys[i] = -1;
    }
}

static int orc_i64_cmp(const void* a, const void* b)
{
    int64_t x = *(const int64_t*)a, y = *(const int64_t*)b;
    return x < y ? -1 : (x > y);
}

static void orc_filter_evict(orc_filter* f)
{
    uint64_t i;
    int64_t first_new = f->n_evict, k;
    if (f->evict_threshold == 0) return;
    for (i = 0; i < f->ts.cap; i++) {
        if (f->ts.state[i] != 1 || f->ts.keys[i] == -1) continue;
        if (f->latest_ts - f->ts.vals[i] > (int64_t)f->evict_threshold) {
            if (f->n_evict == f->evict_cap) {
                f->evict_cap *= 2;
                f->evict_keys = (int64_t*)realloc(f->evict_keys, (size_t)f->evict_cap * sizeof(int64_t));
            }
            f->evict_keys[f->n_evict++] = f->ts.keys[i];
        }
    }
    qsort(f->evict_keys + first_new, (size_t)(f->n_evict - first_new), sizeof(int64_t), orc_i64_cmp);
    /* the reference erases every key in the (accumulated) evict list */
    for (k = 0; k < f->n_evict; k++) {
        orc_map_erase(&f->ts, f->evict_keys[k]);
        if (f->admit_threshold != -1) orc_map_erase(&f->count, f->evict_keys[k]);
    }
}

void orc_filter_record_timestamp(void* h, const int64_t* keys, const int64_t* ts, int64_t n)
{
    orc_filter* f = (orc_filter*)h;
    int64_t i;
    for (i = 0; i < n; i++) {
        orc_map_put(&f->ts, keys[i], ts[i]);
        if (ts[i] > f->latest_ts) f->latest_ts = ts[i];
    }
    if (f->record_batch_id > 0 && (f->record_batch_id + 1) % f->evict_interval == 0) orc_filter_evict(f);
    f->record_batch_id++;
}

int64_t orc_filter_num_evict(void* h) { return ((orc_filter*)h)->n_evict; }
void orc_filter_get_evict(void* h, int64_t* out)
{
    orc_filter* f = (orc_filter*)h;
    memcpy(out, f->evict_keys, (size_t)f->n_evict * sizeof(int64_t));
}
void orc_filter_clear_evict(void* h) { ((orc_filter*)h)->n_evict = 0; }
int64_t orc_filter_count_of(void* h, int64_t key)
{
    int64_t* hit = orc_map_find(&((orc_filter*)h)->count, key);
    return hit ? *hit : -1;
}

/* ------------------------------------------------------------------------- */
/* A6  pooled embedding gather (forward)                                      */
/* ascendc_op/ai_core_op/split_embedding_codegen_forward_unweighted/v220/     */
/* op_kernel/split_embedding_codegen_forward_unweighted_kernel.h:226-241      */
/* (Pooling: sequential Add from zero, MEAN multiplies by 1.0f/len),          */
/* :316-343 (bag (t,b) -> out[b, D_offsets[t]..]), :299-314 (no pooling),     */
/* README.md:80-124 (numpy statement).  Bags are summed in index order.       */
/* pooling_mode: 0 SUM, 1 MEAN, 2 NONE.                                       */
/* ------------------------------------------------------------------------- */
void orc_tbe_forward(const float* weights, const int64_t* weights_offsets, const int32_t* D_offsets,
                     const int64_t* indices, const int64_t* offsets, int64_t T, int64_t B, int32_t total_D,
                     int32_t max_D, int pooling_mode, float* out)
{
    int64_t t;
    if (pooling_mode == 2) {
#pragma omp parallel for schedule(dynamic, 1)
        for (t = 0; t < T; t++) {
            int64_t s = offsets[t * B], e = offsets[(t + 1) * B], i;
            int32_t D = D_offsets[t + 1] - D_offsets[t];
            for (i = s; i < e; i++) {
                const float* row = weights + weights_offsets[t] + indices[i] * D;
                memset(out + i * max_D, 0, (size_t)max_D * sizeof(float));
                memcpy(out + i * max_D, row, (size_t)D * sizeof(float));
            }
        }
        return;
    }
#pragma omp parallel for collapse(2) schedule(static)
    for (t = 0; t < T; t++) {
        for (int64_t b = 0; b < B; b++) {
            int64_t s = offsets[t * B + b], e = offsets[t * B + b + 1], i;
            int32_t D = D_offsets[t + 1] - D_offsets[t], d;
            float* o = out + b * total_D + D_offsets[t];
            float mean = 1.0f / (float)(e - s);
            for (d = 0; d < D; d++) o[d] = 0.0f;
            for (i = s; i < e; i++) {
                const float* row = weights + weights_offsets[t] + indices[i] * D;
                for (d = 0; d < D; d++) o[d] = o[d] + row[d];
            }
            if (pooling_mode == 1 && e > s)
                for (d = 0; d < D; d++) o[d] = o[d] * mean;
        }
    }
}

/* ------------------------------------------------------------------------- */
/* A7  fused backward: gradient segment-sum over unique rows + optimizer      */
/* ascendc_op/ai_core_op/backward_codegen_adagrad_unweighted_exact/v220/      */
/*  op_kernel/backward_codegen_unweighted_exact_kernel_unique.h:113-148       */
/*    (ComputeGradBag: grad row of bag (t,b), MEAN scales by 1/len, added to  */
/*     G[inverse[i] + unique_offset[t]]), :150-178 (no-bag), :225-268;        */
/*  op_kernel/backward_codegen_adagrad_unweighted_exact_kernel_unique.h:50-62 */
/*    (ComputeAdagrad), ..._adam_..._kernel_unique.h:70-96 (ComputeAdam),     */
/*  op_kernel/backward_codegen_sgd_unweighted_exact_kernel.h:107-124 (SGD),   */
/*  op_host/backward_codegen_adagrad_unweighted_exact.cpp:84-111 (Adam host   */
/*    scalars).                                                               */
/* The reference accumulates G with atomics (unordered); this restatement     */
/* fixes the order to ascending index position, which is the deterministic    */
/* mode of the CUDA path.  optimizer: 1 ADAGRAD, 2 ADAM, 3 SGD.               */
/* ------------------------------------------------------------------------- */
void orc_adam_host_scalars(float beta1, float beta2, int64_t iter, float* beta2sqrt_out)
{
    float b1 = (float)(1 - pow((double)beta1, (double)iter));
    float b2 = (float)(1 - pow((double)beta2, (double)iter));
    *beta2sqrt_out = (float)(sqrt((double)b2) / (double)b1);
}

static void orc_update_row(int optimizer, float* w, float* m1, float* m2, const float* g, int32_t D, float lr,
                           float eps, float beta1, float beta2, float beta2sqrt)
{
    int32_t d;
    if (optimizer == 1) {
        for (d = 0; d < D; d++) {
            float g2 = g[d] * g[d];
            float s = m1[d] + g2;
            float den = sqrtf(s) + eps;
            float q = lr / den;
            float delta = (q * g[d]) * -1.0f;
            w[d] = w[d] + delta;
            m1[d] = m1[d] + g2;
        }
    } else if (optimizer == 2) {
        float omb1 = 1 - beta1, omb2 = 1 - beta2;
        float step = (-lr) * beta2sqrt;
        for (d = 0; d < D; d++) {
            float a = m1[d] * beta1;
            float b = g[d] * omb1;
            float nm1 = a + b;
            float c = m2[d] * beta2;
            float e = (g[d] * g[d]) * omb2;
            float nm2 = c + e;
            float den = sqrtf(nm2) + eps;
            float delta = (nm1 / den) * step;
            w[d] = w[d] + delta;
            m1[d] = nm1;
            m2[d] = nm2;
        }
    } else {
        for (d = 0; d < D; d++) w[d] = w[d] + g[d] * (-lr);
    }
}

/* unique_ids / unique_offsets / unique_inverse may be NULL: the op then
 * dedups internally on hash_size_cumsum[t] + idx (same result). */
int orc_tbe_backward(const float* grad_output, float* weights, float* momentum1, float* momentum2,
                     const int64_t* weights_offsets, const int32_t* D_offsets, const int64_t* hash_size_cumsum,
                     const int64_t* indices, const int64_t* offsets, const int64_t* unique_ids,
                     const int64_t* unique_offsets, const int64_t* unique_inverse, int64_t T, int64_t B,
                     int32_t total_D, int32_t max_D, int pooling_mode, int optimizer, float lr, float eps,
                     float beta1, float beta2, int64_t iter, int gradient_clipping, float max_gradient,
                     int reduce_chunk)
{
    int64_t N = offsets[T * B];
    int64_t U, t, u, i;
    int64_t *own_uid = NULL, *own_uoff = NULL, *own_inv = NULL;
    float beta2sqrt = 0.0f;
    float* G;
    if (optimizer == 2) orc_adam_host_scalars(beta1, beta2, iter, &beta2sqrt);
    if (!unique_ids) {
        /* internal dedup: one merged sorted-unique over linearised rows; a
         * feature f then uses offset 0 and the linear index (hash_size_cumsum
         * makes features of one table share rows). */
        int64_t* lin = (int64_t*)malloc((size_t)(N > 0 ? N : 1) * sizeof(int64_t));
        own_uid = (int64_t*)malloc((size_t)(N > 0 ? N : 1) * sizeof(int64_t));
        own_inv = (int64_t*)malloc((size_t)(N > 0 ? N : 1) * sizeof(int64_t));
        for (t = 0; t < T; t++)
            for (i = offsets[t * B]; i < offsets[(t + 1) * B]; i++) lin[i] = hash_size_cumsum[t] + indices[i];
        U = orc_unique_sorted(lin, N, own_uid, own_inv);
        free(lin);
    } else {
        U = unique_offsets[T];
    }
    /* malloc + memset, not calloc: the pages are touched here, by one thread, instead of faulting in from all
     * threads at once inside the parallel walk below */
    G = (float*)malloc((size_t)(U > 0 ? U : 1) * (size_t)max_D * sizeof(float));
    memset(G, 0, (size_t)(U > 0 ? U : 1) * (size_t)max_D * sizeof(float));
    /* (1) segment-sum in ascending index position.  reduce_chunk == 0: one
     * sequential sum.  reduce_chunk == C: a row with more than C contributions
     * sums consecutive chunks of C contributions (each from 0.0f) and then the
     * chunk sums (from 0.0f), both in order. */
    {
        const int64_t* inv = unique_ids ? unique_inverse : own_inv;
        int64_t* cnt = (int64_t*)calloc((size_t)(U > 0 ? U : 1), sizeof(int64_t));
        int64_t* seen = (int64_t*)calloc((size_t)(U > 0 ? U : 1), sizeof(int64_t));
        float* P = (float*)malloc((size_t)(U > 0 ? U : 1) * (size_t)max_D * sizeof(float)); /* open chunk */
        memset(P, 0, (size_t)(U > 0 ? U : 1) * (size_t)max_D * sizeof(float));
        if (reduce_chunk > 0)
            for (t = 0; t < T; t++) {
                int64_t uoff = unique_ids ? unique_offsets[t] : 0;
                for (i = offsets[t * B]; i < offsets[(t + 1) * B]; i++) cnt[inv[i] + uoff]++;
            }
        /* The order of additions is what fixes the result, and it is per unique row: the contributions of a
         * row are taken in ascending index position.  Threads therefore own disjoint sets of unique rows
         * (row u belongs to thread u mod nth); every thread walks all indices in the serial order and performs
         * the additions of its own rows only, so each row sees exactly the serial sequence of additions.
         * Whether index i closes a chunk is integer bookkeeping, resolved once beforehand. */
        {
            unsigned char* closes = (unsigned char*)calloc((size_t)(N > 0 ? N : 1), 1);
            if (reduce_chunk > 0)
                for (t = 0; t < T; t++) {
                    int64_t uoff = unique_ids ? unique_offsets[t] : 0;
                    for (i = offsets[t * B]; i < offsets[(t + 1) * B]; i++) {
                        int64_t u2 = inv[i] + uoff;
                        if (cnt[u2] > reduce_chunk) {
                            seen[u2]++;
                            closes[i] = (unsigned char)((seen[u2] % reduce_chunk == 0 || seen[u2] == cnt[u2]) ? 2 : 1);
                        }
                    }
                }
#pragma omp parallel
            {
                int nth = 1, tid = 0;
                int64_t tt, ii;
#ifdef _OPENMP
                nth = omp_get_num_threads();
                tid = omp_get_thread_num();
#endif
                for (tt = 0; tt < T; tt++) {
                    int32_t D = D_offsets[tt + 1] - D_offsets[tt], d;
                    const int32_t d_lo = 0, d_hi = D;
                    int64_t b;
                    int64_t uoff = unique_ids ? unique_offsets[tt] : 0;
                    for (b = 0; b < B; b++) {
                        int64_t s0 = offsets[tt * B + b], e0 = offsets[tt * B + b + 1];
                        float mean = 1.0f / (float)(e0 - s0);
                        for (ii = s0; ii < e0; ii++) {
                            const float* g = pooling_mode == 2 ? grad_output + ii * max_D
                                                               : grad_output + b * total_D + D_offsets[tt];
                            int64_t u2 = inv[ii] + uoff;
                            int chunked = closes[ii] != 0;
                            float* acc;
                            if (u2 % nth != tid) continue;
                            acc = chunked ? P + u2 * max_D : G + u2 * max_D;
                            for (d = d_lo; d < d_hi; d++) {
                                float v = g[d];
                                if (gradient_clipping)
                                    v = v < -max_gradient ? -max_gradient : (v > max_gradient ? max_gradient : v);
                                if (pooling_mode == 1) v = v * mean;
                                acc[d] = acc[d] + v;
                            }
                            if (closes[ii] == 2) { /* chunk closed */
                                float* tot = G + u2 * max_D;
                                for (d = d_lo; d < d_hi; d++) {
                                    tot[d] = tot[d] + acc[d];
                                    acc[d] = 0.0f;
                                }
                            }
                        }
                    }
                }
            }
            free(closes);
        }
        free(cnt);
        free(seen);
        free(P);
    }
    /* (2) one update per unique row */
    if (unique_ids) {
        for (t = 0; t < T; t++) {
            /* ranges repeat for features of one table; update a range once
             * (AdagradScheduler/AdamScheduler: skip when the bound repeats) */
            int32_t D = D_offsets[t + 1] - D_offsets[t];
            if (t + 1 < T && unique_offsets[t + 1] == unique_offsets[t]) continue;
            if (unique_offsets[t + 1] == unique_offsets[t]) continue;
#pragma omp parallel for schedule(static)
            for (u = unique_offsets[t]; u < unique_offsets[t + 1]; u++) {
                int64_t r = weights_offsets[t] + unique_ids[u] * D;
                orc_update_row(optimizer, weights + r, momentum1 ? momentum1 + r : NULL,
                               momentum2 ? momentum2 + r : NULL, G + u * max_D, D, lr, eps, beta1, beta2, beta2sqrt);
            }
        }
    } else {
#pragma omp parallel for schedule(static)
        for (u = 0; u < U; u++) {
            int64_t lin = own_uid[u], f = -1, r, ff;
            int32_t D;
            /* the table that holds linear row `lin` starts at the largest hash_size_cumsum[f] <= lin; entries
             * repeat (and are not monotonic in f) when features share tables, so look at all of them */
            for (ff = 0; ff < T; ff++)
                if (hash_size_cumsum[ff] <= lin && (f < 0 || hash_size_cumsum[ff] > hash_size_cumsum[f])) f = ff;
            if (f < 0) continue;
            D = D_offsets[f + 1] - D_offsets[f];
            r = weights_offsets[f] + (lin - hash_size_cumsum[f]) * D;
            orc_update_row(optimizer, weights + r, momentum1 ? momentum1 + r : NULL, momentum2 ? momentum2 + r : NULL,
                           G + u * max_D, D, lr, eps, beta1, beta2, beta2sqrt);
        }
    }
    free(G);
    free(own_uid);
    free(own_uoff);
    free(own_inv);
    return ORC_OK;
}

/* ------------------------------------------------------------------------- */
/* A8  row gather / row assign by slot (swap-in / swap-out helpers)           */
/* hybrid_torchrec/distributed/batched_embedding_kernel.py:297-345            */
/* ------------------------------------------------------------------------- */
void orc_gather_rows(const float* table, const int64_t* slots, int64_t k, int32_t D, float* out)
{
    int64_t i;
    for (i = 0; i < k; i++) memcpy(out + i * D, table + slots[i] * D, (size_t)D * sizeof(float));
}

void orc_scatter_rows(float* table, const int64_t* slots, int64_t k, int32_t D, const float* rows)
{
    int64_t i;
    for (i = 0; i < k; i++) memcpy(table + slots[i] * D, rows + i * D, (size_t)D * sizeof(float));
}

/* ------------------------------------------------------------------------- */
/* A9  TF-flavour ops                                                         */
/* lookup/update by address: ascendc_op/ai_core_op/cust_op_by_addr/v220/      */
/*   op_kernel/embedding_lookup_by_address.cpp:106-145 (address 0 -> zeros),  */
/*   embedding_update_by_address.cpp:100-190 (update_type 0 add, else assign; */
/*   address 0 skipped).  Addresses are element pointers into host memory     */
/*   here (device pointers on the GPU).                                       */
/* LazyAdam: ascendc_op/ai_core_op/fused_lazy_adam/v220/op_kernel/            */
/*   lazy_adam.cpp:138-207; golden cust_op/test/aclnn_lazy_adam_test/tf/      */
/*   scripts/gen_data.py:90-128.  Negative index -> skipped.                  */
/* SGD: ascendc_op/ai_core_op/fused_sgd/v220/op_kernel/sgd_kernel.h:78-190.   */
/* ------------------------------------------------------------------------- */
void orc_lookup_by_address(const int64_t* addresses, int64_t n, int32_t dim, float* out)
{
    int64_t i;
    for (i = 0; i < n; i++) {
        if (addresses[i] != 0)
            memcpy(out + i * dim, (const float*)(intptr_t)addresses[i], (size_t)dim * sizeof(float));
        else
            memset(out + i * dim, 0, (size_t)dim * sizeof(float));
    }
}

void orc_update_by_address(const int64_t* addresses, int64_t n, int32_t dim, const float* rows, int update_type)
{
    int64_t i;
    int32_t d;
    for (i = 0; i < n; i++) {
        float* dst = (float*)(intptr_t)addresses[i];
        if (!dst) continue;
        if (update_type == 0)
            for (d = 0; d < dim; d++) dst[d] = dst[d] + rows[i * dim + d];
        else
            memcpy(dst, rows + i * dim, (size_t)dim * sizeof(float));
    }
}

void orc_lazy_adam(const float* grad, const int32_t* indices, int64_t n, int32_t dim, float* m, float* v, float* var,
                   float lr, float beta1, float beta2, float eps)
{
    int64_t i;
    int32_t d;
    float omb1 = 1 - beta1, omb2 = 1 - beta2, nlr = -lr;
    for (i = 0; i < n; i++) {
        int64_t r = indices[i];
        if (r < 0) continue;
        for (d = 0; d < dim; d++) {
            float g = grad[i * dim + d];
            float a = m[r * dim + d] * beta1;
            float b = g * omb1;
            float nm = a + b;
            float c = v[r * dim + d] * beta2;
            float e = (g * g) * omb2;
            float nv = fabsf(c + e);
            float den = sqrtf(nv) + eps;
            float upd = (nm * nlr) / den;
            m[r * dim + d] = nm;
            v[r * dim + d] = nv;
            var[r * dim + d] = upd + var[r * dim + d];
        }
    }
}

void orc_sgd(const float* grad, const int64_t* indices, int64_t n, int32_t dim, float* var, float lr,
             float weight_decay, int use_weight_decay)
{
    /* the reference gathers every row first, then scatter-adds: duplicated
     * indices see the ORIGINAL var in the weight-decay term */
    int64_t i;
    int32_t d;
    float nlr = -lr;
    float* upd = (float*)malloc((size_t)(n > 0 ? n : 1) * (size_t)dim * sizeof(float));
    for (i = 0; i < n; i++) {
        int64_t r = indices[i];
        for (d = 0; d < dim; d++) {
            float g = grad[i * dim + d];
            if (use_weight_decay && r >= 0) g = g + var[r * dim + d] * weight_decay;
            upd[i * dim + d] = g * nlr;
        }
    }
    for (i = 0; i < n; i++) {
        int64_t r = indices[i];
        if (r < 0) continue;
        for (d = 0; d < dim; d++) var[r * dim + d] = var[r * dim + d] + upd[i * dim + d];
    }
    free(upd);
}

/* ------------------------------------------------------------------------- */
/* A10 Restore: hash_indices[r] = unique_indices[inverse[r] + unique_offset[t]]*/
/* torchrec_embcache/csrc/ops/restore.cpp:15-51                               */
/* ------------------------------------------------------------------------- */
void orc_restore(const int64_t* unique_indices, const int64_t* unique_inverse, const int64_t* unique_offset,
                 const int64_t* offsets_per_table, int64_t n_tables, int64_t* hash_indices)
{
    int64_t t, r;
    for (t = 0; t < n_tables; t++)
        for (r = offsets_per_table[t]; r < offsets_per_table[t + 1]; r++)
            hash_indices[r] = unique_indices[unique_inverse[r] + unique_offset[t]];
}
