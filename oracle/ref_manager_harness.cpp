// TEST INFRASTRUCTURE ONLY -- never linked into or called by the product path.
//
// A flat C ABI over the reference's own `Embcache::EmbcacheManager` for the host tier and the checkpoint
// files: rows are put into its host store with EmbeddingUpdate (InsertOrAssign of caller-given rows; the
// lookup path allocates pinned tensors and needs a GPU driver, so it is not used), written with Save and read
// with Load.  Compiled together with the reference sources where they lie (recipe: oracle/build_ref.py);
// nothing of the reference is copied here, only its public class interface is called.
#include <cstdint>
#include <exception>
#include <string>
#include <vector>

#include <torch/torch.h>

#include "embedding_cache/embcache_manager.h"
#include "utils/logger.h"

using namespace Embcache;

extern "C" {

void* refmgr_new(const char* table_name, int32_t dim, int32_t optim_num, int64_t cache_size, float init_min,
                 float init_max, int64_t admit_threshold, uint64_t evict_threshold, uint64_t evict_step_interval)
{
    try {
        EmbConfig cfg;
        cfg.tableName = table_name;
        cfg.initializerType = InitializerType::LINEAR;
        cfg.embDim = dim;
        cfg.optimNum = optim_num;
        cfg.cacheSize = cache_size;
        cfg.weightInitMin = init_min;
        cfg.weightInitMax = init_max;
        cfg.weightInitMean = 0.f;
        cfg.weightInitStddev = 1.f;
        cfg.admitAndEvictConfig = AdmitAndEvictConfig(admit_threshold, 0.f, evict_threshold, evict_step_interval);
        cfg.initializerRandomPoolSize = -1;
        cfg.seed = 0;
        return new EmbcacheManager(std::vector<EmbConfig>{cfg}, true);
    } catch (const std::exception&) {
        return nullptr;
    }
}

void refmgr_free(void* h) { delete static_cast<EmbcacheManager*>(h); }

// InsertOrAssign of n rows: embs / m1 / m2 are [n, dim] (m1, m2 as many as optim_num)
int refmgr_update(void* h, const int64_t* keys, int64_t n, int32_t dim, float* embs, float* m1, float* m2)
{
    try {
        auto* m = static_cast<EmbcacheManager*>(h);
        SwapInfo info;
        info.swapoutKeys = {std::vector<int64_t>(keys, keys + n)};
        auto e = torch::from_blob(embs, {n * dim}, torch::kFloat32);
        std::vector<at::Tensor> optims;
        if (m1) optims.push_back(torch::from_blob(m1, {n * dim}, torch::kFloat32));
        if (m2) optims.push_back(torch::from_blob(m2, {n * dim}, torch::kFloat32));
        m->EmbeddingUpdateAsync(info, e, optims, {}).get();  // the public entry; runs EmbeddingUpdate on a pool thread
        return 0;
    } catch (const std::exception&) {
        return -1;
    }
}

// StatisticsKeyCount for table 0 (admission counts, saved with the checkpoint)
int refmgr_statistics(void* h, int64_t* keys, int64_t n)
{
    try {
        auto* m = static_cast<EmbcacheManager*>(h);
        auto k = torch::from_blob(keys, {n}, torch::kInt64);
        auto off = torch::tensor(std::vector<int64_t>{0, n}, torch::kInt64);
        m->StatisticsKeyCount(k, off, torch::empty({0}, torch::kInt64), 0);
        return 0;
    } catch (const std::exception&) {
        return -1;
    }
}

int refmgr_record_timestamp(void* h, int64_t* keys, int64_t* ts, int64_t n)
{
    try {
        auto* m = static_cast<EmbcacheManager*>(h);
        m->RecordTimestamp(torch::from_blob(keys, {n}, torch::kInt64), {0, n}, torch::from_blob(ts, {n}, torch::kInt64), {});
        return 0;
    } catch (const std::exception&) {
        return -1;
    }
}

int refmgr_save(void* h, const char* path, int rank)
{
    try {
        static_cast<EmbcacheManager*>(h)->Save(path, rank);
        return 0;
    } catch (const std::exception&) {
        return -1;
    }
}

int refmgr_load(void* h, const char* path, int rank)
{
    try {
        static_cast<EmbcacheManager*>(h)->Load(path, rank);
        return 0;
    } catch (const std::exception&) {
        return -1;
    }
}

}  // extern "C"
