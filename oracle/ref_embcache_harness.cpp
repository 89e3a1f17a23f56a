// TEST INFRASTRUCTURE ONLY -- never linked into or called by the product path.
//
// A flat C ABI over the reference's own `Embcache::SwapManager` and
// `Embcache::FeatureFilter` classes so the parity tests and the CPU baseline
// can drive the unmodified reference slot policy through ctypes.
//
// This file is compiled together with the reference sources where they lie:
//   torchrec_embcache/csrc/embedding_cache/swap_manager.cpp
//   torchrec_embcache/csrc/feature_filter/feature_filter.cpp
//   torchrec_embcache/csrc/feature_filter/evict_feature_record.cpp
//   torchrec_embcache/csrc/utils/logger.cpp
// (recipe: oracle/build_ref.py).  Nothing of the reference is copied here;
// only its public class interface is called.
#include <cstdint>
#include <cstring>
#include <exception>
#include <string>
#include <vector>

#include "embedding_cache/swap_manager.h"
#include "feature_filter/feature_filter.h"
#include "utils/logger.h"

using Embcache::FeatureFilter;
using Embcache::SwapManager;

extern "C" {

void ref_set_log_level(int level) { Embcache::Logger::SetLevel(level); }

void* ref_swap_new(int64_t cache_size, int64_t mem_start_offset)
{
    return new SwapManager(cache_size, mem_start_offset);
}

void ref_swap_free(void* h) { delete static_cast<SwapManager*>(h); }

// Output arrays must hold n entries each.  Returns 0, or -1 when the reference
// throws ("cacheSize_ too small").
int ref_swap_compute(void* h, const int64_t* keys, int64_t n, int64_t* batch_offs,
                     int64_t* swapin_keys, int64_t* swapin_offs, int64_t* n_swapin,
                     int64_t* swapout_keys, int64_t* swapout_offs, int64_t* n_swapout)
{
    auto* sm = static_cast<SwapManager*>(h);
    std::vector<int64_t> k(keys, keys + n);
    try {
        auto ret = sm->ComputeSwapInfo(k);
        const auto& so_k = std::get<0>(ret);
        const auto& so_o = std::get<1>(ret);
        const auto& si_k = std::get<2>(ret);
        const auto& si_o = std::get<3>(ret);
        const auto& bo = std::get<4>(ret);
        if (!bo.empty()) std::memcpy(batch_offs, bo.data(), bo.size() * sizeof(int64_t));
        if (!si_k.empty()) std::memcpy(swapin_keys, si_k.data(), si_k.size() * sizeof(int64_t));
        if (!si_o.empty()) std::memcpy(swapin_offs, si_o.data(), si_o.size() * sizeof(int64_t));
        if (!so_k.empty()) std::memcpy(swapout_keys, so_k.data(), so_k.size() * sizeof(int64_t));
        if (!so_o.empty()) std::memcpy(swapout_offs, so_o.data(), so_o.size() * sizeof(int64_t));
        *n_swapin = static_cast<int64_t>(si_k.size());
        *n_swapout = static_cast<int64_t>(so_k.size());
        return 0;
    } catch (const std::exception&) {
        return -1;
    }
}

void ref_swap_remove(void* h, const int64_t* keys, int64_t n)
{
    std::vector<int64_t> k(keys, keys + n);
    static_cast<SwapManager*>(h)->RemoveKeys(k);
}

int64_t ref_swap_occupied(void* h) { return static_cast<SwapManager*>(h)->GetOccupiedNum(); }

void* ref_filter_new(int64_t admit_threshold, uint64_t evict_threshold, uint64_t evict_step_interval)
{
    return new FeatureFilter(std::string("t"), admit_threshold, evict_threshold, evict_step_interval);
}

void ref_filter_free(void* h) { delete static_cast<FeatureFilter*>(h); }

void ref_filter_statistics(void* h, const int64_t* keys, const int64_t* counts, int64_t n)
{
    static_cast<FeatureFilter*>(h)->StatisticsKeyCount(keys, counts, 0, n, counts == nullptr);
}

void ref_filter_count_filter(void* h, int64_t* keys_inout, int64_t n)
{
    static_cast<FeatureFilter*>(h)->CountFilter(keys_inout, 0, n);
}

void ref_filter_record_timestamp(void* h, const int64_t* keys, const int64_t* ts, int64_t n)
{
    static_cast<FeatureFilter*>(h)->RecordTimestamp(keys, 0, n, ts);
}

int64_t ref_filter_num_evict(void* h)
{
    return static_cast<int64_t>(static_cast<FeatureFilter*>(h)->evictFeatureRecord_.GetEvictKeys().size());
}

void ref_filter_get_evict(void* h, int64_t* out)
{
    const auto& v = static_cast<FeatureFilter*>(h)->evictFeatureRecord_.GetEvictKeys();
    if (!v.empty()) std::memcpy(out, v.data(), v.size() * sizeof(int64_t));
}

void ref_filter_clear_evict(void* h) { static_cast<FeatureFilter*>(h)->evictFeatureRecord_.ClearEvictInfo(); }

int64_t ref_filter_count_of(void* h, int64_t key)
{
    const auto& m = static_cast<FeatureFilter*>(h)->GetFeatureCountMap();
    auto it = m.find(key);
    return it == m.end() ? -1 : static_cast<int64_t>(it->second.count);
}

}  // extern "C"
