// Host (DRAM) tier of the hybrid cache: key -> row store for the embedding rows that do not fit, or are not
// currently held in, the HBM cache.  Host code only (no kernel): the device side of a swap is recsdk_gather_rows /
// recsdk_scatter_rows plus asynchronous copies between pinned staging buffers and the GPU, driven by the caller.
//
// Semantics of Embcache::EmbTable (torchrec_embcache/csrc/emb_table/emb_table.h:32-372):
//   rows are AoS [w | m | v] of width (1 + optim_num) * emb_dim (:34-37);
//   FindOrInsert   a missing key gets a new row: weights from the configured initializer, optimizer state zero; the
//                  row is then copied out into SoA output arrays (one [n, emb_dim] block per array) (:54-116, :218-277)
//   InsertOrAssign creates the row when missing (no initializer) and overwrites it from SoA inputs (:118-179)
//   RemoveEmbedding, ForEachKey (:300-330)
// Initializers (emb_table/initializer.h): LINEAR = min + i/(dim-1)*(max-min) computed in double (:44-56), UNIFORM over
// [min, max) (:36-42), TRUNCATED_NORMAL with rejection outside [min, max] (:58-75).  The reference seeds the two random
// ones from std::random_device; here they draw from one generator seeded by the caller, so runs repeat.
//
// Storage: open addressing over {key, row index}; rows live in fixed-size slabs so that growing the key table
// never moves a row; removed rows go to a free list.  One mutex per table, as in the reference's map-backed
// table.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <memory>
#include <mutex>
#include <random>
#include <vector>

#include "recsdk_b200.h"

namespace {

constexpr int64_t kEmptyKey = INT64_MIN;
constexpr int64_t kTombKey = INT64_MIN + 1;
constexpr int64_t kSlabRows = 1 << 14;

inline uint64_t mix64(uint64_t x)
{
    x += 0x9e3779b97f4a7c15ull;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
    return x ^ (x >> 31);
}

struct HostTable {
    int32_t D = 0, S = 0, ext = 0, init_type = 0;
    float init_min = 0.f, init_max = 0.f, init_mean = 0.f, init_std = 1.f;
    std::mt19937 gen;
    std::vector<int64_t> keys;  // open addressing, power-of-two capacity
    std::vector<int64_t> rows;  // row index per entry
    std::vector<std::unique_ptr<float[]>> slabs;
    std::vector<int64_t> free_rows;
    int64_t next_row = 0, live = 0, used = 0;  // used = live + tombstones
    std::mutex mu;

    float* row_ptr(int64_t r) { return slabs[static_cast<size_t>(r / kSlabRows)].get() + (r % kSlabRows) * ext; }

    int64_t find(int64_t key) const
    {
        const uint64_t mask = keys.size() - 1;
        for (uint64_t i = mix64(static_cast<uint64_t>(key)) & mask;; i = (i + 1) & mask) {
            if (keys[i] == key) return static_cast<int64_t>(i);
            if (keys[i] == kEmptyKey) return -1;
        }
    }

    void grow()
    {
        std::vector<int64_t> ok, orw;
        ok.swap(keys);
        orw.swap(rows);
        size_t cap = ok.size();
        while (static_cast<size_t>(live) * 10 >= cap * 5) cap <<= 1;  // rebuilt at <= 50 % load, tombstones dropped
        keys.assign(cap, kEmptyKey);
        rows.assign(cap, -1);
        const uint64_t mask = cap - 1;
        for (size_t j = 0; j < ok.size(); ++j) {
            if (ok[j] == kEmptyKey || ok[j] == kTombKey) continue;
            uint64_t i = mix64(static_cast<uint64_t>(ok[j])) & mask;
            while (keys[i] != kEmptyKey) i = (i + 1) & mask;
            keys[i] = ok[j];
            rows[i] = orw[j];
        }
        used = live;
    }

    // entry of `key`, created (with a fresh, zeroed row) when missing; *created tells which
    int64_t find_or_create(int64_t key, bool* created)
    {
        if (static_cast<size_t>(used + 1) * 10 > keys.size() * 7) grow();
        const uint64_t mask = keys.size() - 1;
        int64_t tomb = -1;
        uint64_t i = mix64(static_cast<uint64_t>(key)) & mask;
        for (;; i = (i + 1) & mask) {
            if (keys[i] == key) {
                *created = false;
                return static_cast<int64_t>(i);
            }
            if (keys[i] == kTombKey && tomb < 0) tomb = static_cast<int64_t>(i);
            if (keys[i] == kEmptyKey) break;
        }
        const int64_t e = tomb >= 0 ? tomb : static_cast<int64_t>(i);
        if (tomb < 0) ++used;
        int64_t r;
        if (!free_rows.empty()) {
            r = free_rows.back();
            free_rows.pop_back();
        } else {
            r = next_row++;
            if (static_cast<size_t>(r / kSlabRows) >= slabs.size())
                slabs.emplace_back(new float[static_cast<size_t>(kSlabRows) * ext]);
        }
        memset(row_ptr(r), 0, sizeof(float) * ext);
        keys[e] = key;
        rows[e] = r;
        ++live;
        *created = true;
        return e;
    }

    void init_weights(float* w)
    {
        if (init_type == RECSDK_HOST_INIT_LINEAR) {
            if (D == 1) {
                w[0] = init_min;
                return;
            }
            for (int32_t i = 0; i < D; ++i) w[i] = static_cast<float>(init_min + 1.0 * i / (D - 1) * (init_max - init_min));
        } else if (init_type == RECSDK_HOST_INIT_TRUNCATED_NORMAL) {
            if (init_std <= 0.f || init_min >= init_max) return;
            std::normal_distribution<float> dist(init_mean, init_std);
            for (int32_t i = 0; i < D; ++i) {
                float v = dist(gen);
                while (v < init_min || v > init_max) v = dist(gen);
                w[i] = v;
            }
        } else {
            std::uniform_real_distribution<float> dist(init_min, init_max);
            for (int32_t i = 0; i < D; ++i) w[i] = dist(gen);
        }
    }
};

inline HostTable* as_table(recsdk_host_table* t) { return reinterpret_cast<HostTable*>(t); }

}  // namespace

extern "C" recsdk_host_table* recsdk_host_table_create(int32_t emb_dim, int32_t optim_num, int32_t initializer_type,
                                                       float weight_init_min, float weight_init_max,
                                                       float weight_init_mean, float weight_init_stddev, int64_t seed,
                                                       int64_t reserve_rows)
{
    if (emb_dim <= 0 || optim_num < 0 || optim_num > 2) return nullptr;
    if (initializer_type < RECSDK_HOST_INIT_LINEAR || initializer_type > RECSDK_HOST_INIT_UNIFORM) return nullptr;
    HostTable* t = new (std::nothrow) HostTable();
    if (t == nullptr) return nullptr;
    t->D = emb_dim;
    t->S = optim_num;
    t->ext = (1 + optim_num) * emb_dim;
    t->init_type = initializer_type;
    t->init_min = weight_init_min;
    t->init_max = weight_init_max;
    t->init_mean = weight_init_mean;
    t->init_std = weight_init_stddev;
    t->gen.seed(static_cast<uint32_t>(seed));
    size_t cap = 1024;
    while (cap < static_cast<size_t>(reserve_rows > 0 ? reserve_rows : 0) * 2) cap <<= 1;
    t->keys.assign(cap, kEmptyKey);
    t->rows.assign(cap, -1);
    return reinterpret_cast<recsdk_host_table*>(t);
}

extern "C" void recsdk_host_table_destroy(recsdk_host_table* t) { delete as_table(t); }

extern "C" int64_t recsdk_host_table_size(recsdk_host_table* t)
{
    if (t == nullptr) return -1;
    std::lock_guard<std::mutex> lk(as_table(t)->mu);
    return as_table(t)->live;
}

extern "C" int recsdk_host_table_find_or_insert(recsdk_host_table* t, const int64_t* keys, int64_t n, float* out_embs,
                                                float* out_optim1, float* out_optim2)
{
    HostTable* h = as_table(t);
    if (h == nullptr || n < 0 || (n > 0 && (keys == nullptr || out_embs == nullptr))) return RECSDK_ERR_INVALID_ARG;
    if ((h->S > 0 && n > 0 && out_optim1 == nullptr) || (h->S > 1 && n > 0 && out_optim2 == nullptr))
        return RECSDK_ERR_INVALID_ARG;
    std::lock_guard<std::mutex> lk(h->mu);
    const size_t bytes = sizeof(float) * h->D;
    for (int64_t i = 0; i < n; ++i) {
        if (keys[i] == kEmptyKey || keys[i] == kTombKey) return RECSDK_ERR_INVALID_ARG;
        bool created;
        const int64_t e = h->find_or_create(keys[i], &created);
        float* row = h->row_ptr(h->rows[e]);
        if (created) h->init_weights(row);
        memcpy(out_embs + i * h->D, row, bytes);
        if (h->S > 0) memcpy(out_optim1 + i * h->D, row + h->D, bytes);
        if (h->S > 1) memcpy(out_optim2 + i * h->D, row + 2 * h->D, bytes);
    }
    return RECSDK_OK;
}

extern "C" int recsdk_host_table_insert_or_assign(recsdk_host_table* t, const int64_t* keys, int64_t n,
                                                  const float* in_embs, const float* in_optim1, const float* in_optim2)
{
    HostTable* h = as_table(t);
    if (h == nullptr || n < 0 || (n > 0 && (keys == nullptr || in_embs == nullptr))) return RECSDK_ERR_INVALID_ARG;
    if ((h->S > 0 && n > 0 && in_optim1 == nullptr) || (h->S > 1 && n > 0 && in_optim2 == nullptr))
        return RECSDK_ERR_INVALID_ARG;
    std::lock_guard<std::mutex> lk(h->mu);
    const size_t bytes = sizeof(float) * h->D;
    for (int64_t i = 0; i < n; ++i) {
        if (keys[i] == kEmptyKey || keys[i] == kTombKey) return RECSDK_ERR_INVALID_ARG;
        bool created;
        const int64_t e = h->find_or_create(keys[i], &created);
        float* row = h->row_ptr(h->rows[e]);
        memcpy(row, in_embs + i * h->D, bytes);
        if (h->S > 0) memcpy(row + h->D, in_optim1 + i * h->D, bytes);
        if (h->S > 1) memcpy(row + 2 * h->D, in_optim2 + i * h->D, bytes);
    }
    return RECSDK_OK;
}

extern "C" int recsdk_host_table_remove(recsdk_host_table* t, const int64_t* keys, int64_t n)
{
    HostTable* h = as_table(t);
    if (h == nullptr || n < 0 || (n > 0 && keys == nullptr)) return RECSDK_ERR_INVALID_ARG;
    std::lock_guard<std::mutex> lk(h->mu);
    for (int64_t i = 0; i < n; ++i) {
        const int64_t e = h->find(keys[i]);
        if (e < 0) continue;
        h->free_rows.push_back(h->rows[e]);
        h->keys[e] = kTombKey;
        h->rows[e] = -1;
        --h->live;
    }
    return RECSDK_OK;
}

extern "C" int64_t recsdk_host_table_export(recsdk_host_table* t, int64_t* keys_out, float* embs_out, float* optim1_out,
                                            float* optim2_out, int64_t capacity)
{
    HostTable* h = as_table(t);
    if (h == nullptr) return -1;
    std::lock_guard<std::mutex> lk(h->mu);
    if (keys_out == nullptr) return h->live;
    if (capacity < h->live) return -1;
    const size_t bytes = sizeof(float) * h->D;
    int64_t k = 0;
    for (size_t j = 0; j < h->keys.size(); ++j) {
        if (h->keys[j] == kEmptyKey || h->keys[j] == kTombKey) continue;
        const float* row = h->row_ptr(h->rows[j]);
        keys_out[k] = h->keys[j];
        if (embs_out) memcpy(embs_out + k * h->D, row, bytes);
        if (optim1_out && h->S > 0) memcpy(optim1_out + k * h->D, row + h->D, bytes);
        if (optim2_out && h->S > 1) memcpy(optim2_out + k * h->D, row + 2 * h->D, bytes);
        ++k;
    }
    return k;
}
