// Torch custom-op registration over the C ABI of include/recsdk_b200.h.
//
// Same schema strings as the reference's registration
// (cust_op/framework/torch_plugin/torch_library/2.6.0/split_embedding_codegen_forward_unweighted/
//  split_embedding_codegen_forward_unweighted.cpp:77-95, backward_codegen_adagrad_unweighted_exact.cpp:282-365,
//  backward_codegen_adam_unweighted_exact.cpp:418-505, backward_codegen_sgd_unweighted_exact.cpp:336-417),
// registered under `fbgemm::` (what the reference's invokers call) and, identically, under `recsdk::`
// (usable when a real fbgemm_gpu owns the fbgemm namespace; build with -DRECSDK_NO_FBGEMM_NS then).
// The implementations enqueue the CUDA kernels of librecsdk_b200.so on the current stream; uvm / lxu cache /
// placements / vbe arguments are accepted and ignored, as in the reference.
// Also: class `recsdk::IdsMapper` with the methods of `hybrid::IdsMapper`
// (hybrid_torchrec/src/bind_torch_lib.cpp:9-19) and `recsdk::block_bucketize_sparse_features`.
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>

#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <torch/csrc/autograd/custom_function.h>
#include <torch/custom_class.h>
#include <torch/library.h>
#include <torch/torch.h>

#include "recsdk_b200.h"

namespace recsdk_torch {

using at::Tensor;
using torch::autograd::AutogradContext;
using torch::autograd::variable_list;

static void* cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

static void check_rc(int rc, const char* where) { TORCH_CHECK(rc == RECSDK_OK, where, ": ", recsdk_error_string(rc)); }

static const Tensor& pick(const Tensor& indices, const Tensor& hash_indices)
{
    return (hash_indices.defined() && hash_indices.numel() > 0) ? hash_indices : indices;
}

static void check_i64(const Tensor& t, const char* name)
{
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t.scalar_type() == at::kLong, name, " must be int64");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

// ---------------------------------------------------------------------------- forward
// Set by the lookup function around its own forward when it has just enqueued a plan on the side stream: the
// pooled gather then runs with three resident blocks per SM so that the plan's kernels find SM slots beside it.
static thread_local bool t_forward_leave_room = false;

Tensor forward_unweighted_cuda(const Tensor& dev_weights, const Tensor& uvm_weights, const Tensor& lxu_cache_weights,
                               const Tensor& weights_placements, const Tensor& weights_offsets, const Tensor& D_offsets,
                               c10::SymInt total_D, c10::SymInt max_D, const Tensor& indices, const Tensor& offsets,
                               int64_t pooling_mode, const Tensor& lxu_cache_locations, const Tensor& uvm_cache_stats,
                               int64_t output_dtype, bool is_experimental, const Tensor& hash_indices,
                               const Tensor& offset_per_key)
{
    const int64_t totalD = total_D.guard_int(__FILE__, __LINE__);
    const int64_t maxD = max_D.guard_int(__FILE__, __LINE__);
    TORCH_CHECK(dev_weights.is_cuda(), "dev_weights must be a CUDA tensor (recsdk_b200 has no CPU path)");
    const c10::cuda::OptionalCUDAGuard guard(device_of(dev_weights));
    const int64_t T = weights_offsets.size(0);
    const Tensor& idx = pick(indices, hash_indices);
    if (T == 0 || idx.numel() == 0) return Tensor();  // forward.cpp:49-55
    TORCH_CHECK((offsets.size(0) - 1) % T == 0, "offset size = ", offsets.size(0),
                " is incorrect for feature count = ", T);
    TORCH_CHECK(dev_weights.scalar_type() == at::kFloat && dev_weights.is_contiguous(), "dev_weights must be contiguous fp32");
    TORCH_CHECK(D_offsets.scalar_type() == at::kInt, "D_offsets must be int32");
    check_i64(idx, "indices");
    check_i64(offsets, "offsets");
    check_i64(weights_offsets, "weights_offsets");
    const int64_t B = (offsets.size(0) - 1) / T;
    Tensor out = pooling_mode == RECSDK_POOL_NONE ? at::empty({idx.numel(), maxD}, dev_weights.options())
                                                  : at::empty({B, totalD}, dev_weights.options());
    recsdk_tbe_forward_args a{};
    a.dev_weights = dev_weights.data_ptr<float>();
    a.weights_offsets = weights_offsets.data_ptr<int64_t>();
    a.D_offsets = D_offsets.data_ptr<int32_t>();
    a.indices = idx.data_ptr<int64_t>();
    a.offsets = offsets.data_ptr<int64_t>();
    a.out = out.data_ptr<float>();
    a.T = T;
    a.B = B;
    a.N = idx.numel();
    a.total_D = static_cast<int32_t>(totalD);
    a.max_D = static_cast<int32_t>(maxD);
    a.pooling_mode = static_cast<int32_t>(pooling_mode);
    a.flags = t_forward_leave_room ? RECSDK_FWD_LEAVE_ROOM : 0;
    check_rc(recsdk_tbe_forward(&a, cur_stream()), "split_embedding_codegen_forward_unweighted_cuda");
    return out;
}

// ---------------------------------------------------------------------------- fused backward
struct OptArgs {
    int optimizer;
    double eps = 0, lr = 0, beta1 = 0.9, beta2 = 0.999;
    int64_t iter = 1;
};

// Per table set (device, address of dev_weights): the backward's workspace, grown on demand and kept between calls,
// and -- for plan-ahead -- one high-priority side stream with the two events that order it against the caller's
// stream.  Allocating the ~100 MB workspace, a stream and two events on every call cost more host time than the
// launches themselves.  One lookup of a table set is in flight at a time (forward -> backward alternation), which is
// also what makes a single workspace per table set sufficient.
struct TableSetCache {
    Tensor ws;
    std::optional<c10::cuda::CUDAStream> side;
    std::unique_ptr<at::cuda::CUDAEvent> ready, done;
};
static TableSetCache& table_set_cache(const Tensor& dev_weights)
{
    static std::mutex mu;
    static std::map<std::pair<int, const void*>, TableSetCache> caches;
    std::lock_guard<std::mutex> lk(mu);
    return caches[{static_cast<int>(dev_weights.device().index()), dev_weights.const_data_ptr()}];
}
static Tensor cached_workspace(TableSetCache& c, int64_t bytes, const Tensor& like)
{
    if (!c.ws.defined() || c.ws.numel() < bytes) {
        c.ws = at::empty({bytes}, like.options().dtype(at::kByte));
        if (c.side) c10::cuda::CUDACachingAllocator::recordStream(c.ws.storage().data_ptr(), *c.side);
    }
    return c.ws;
}

// flags / ws / plan_total_D: the split form of the call (RECSDK_BWD_PLAN_ONLY without a gradient, then
// RECSDK_BWD_APPLY_ONLY with the same workspace); 0 / undefined / 0 = the whole backward with its own workspace.
static Tensor backward_exact(const Tensor& grad_output_in, const Tensor& dev_weights, const Tensor& weights_offsets,
                             const Tensor& D_offsets, int64_t max_D, const Tensor& hash_size_cumsum,
                             int64_t total_hash_size_bits, const Tensor& indices, const Tensor& offsets,
                             int64_t pooling_mode, const Tensor& momentum1, const Tensor& momentum2,
                             const Tensor& hash_indices, const Tensor& unique_ids, const Tensor& unique_offsets,
                             const Tensor& unique_inverse, const OptArgs& o, int flags = 0, Tensor ws = Tensor(),
                             int64_t plan_total_D = 0, void* stream = nullptr)
{
    TORCH_CHECK(dev_weights.is_cuda(), "dev_weights must be a CUDA tensor (recsdk_b200 has no CPU path)");
    const c10::cuda::OptionalCUDAGuard guard(device_of(dev_weights));
    const int64_t T = weights_offsets.size(0);
    const Tensor& idx = pick(indices, hash_indices);
    if (T == 0 || idx.numel() == 0) return Tensor();
    const bool plan_only = (flags & RECSDK_BWD_PLAN_ONLY) != 0;
    Tensor grad_output = plan_only ? Tensor() : grad_output_in.contiguous();
    TORCH_CHECK(plan_only || grad_output.scalar_type() == at::kFloat, "grad_output must be fp32");
    check_i64(idx, "indices");
    check_i64(offsets, "offsets");
    const int64_t B = (offsets.size(0) - 1) / T;
    recsdk_tbe_backward_args b{};
    b.grad_output = plan_only ? nullptr : grad_output.data_ptr<float>();
    b.flags = flags;
    b.dev_weights = dev_weights.data_ptr<float>();
    if (o.optimizer != RECSDK_OPT_SGD) b.momentum1 = momentum1.data_ptr<float>();
    if (o.optimizer == RECSDK_OPT_ADAM) b.momentum2 = momentum2.data_ptr<float>();
    b.weights_offsets = weights_offsets.data_ptr<int64_t>();
    b.D_offsets = D_offsets.data_ptr<int32_t>();
    b.hash_size_cumsum = hash_size_cumsum.defined() && hash_size_cumsum.numel() ? hash_size_cumsum.data_ptr<int64_t>() : nullptr;
    b.indices = idx.data_ptr<int64_t>();
    b.offsets = offsets.data_ptr<int64_t>();
    const bool have_unique = unique_ids.defined() && unique_ids.numel() > 0;
    if (have_unique) {
        check_i64(unique_ids, "unique_ids");
        check_i64(unique_offsets, "unique_offsets");
        check_i64(unique_inverse, "unique_inverse");
        b.unique_ids = unique_ids.data_ptr<int64_t>();
        b.unique_offsets = unique_offsets.data_ptr<int64_t>();
        b.unique_inverse = unique_inverse.data_ptr<int64_t>();
        b.num_unique_capacity = unique_ids.numel();
    }
    b.T = T;
    b.B = B;
    b.N = idx.numel();
    b.total_D = static_cast<int32_t>(pooling_mode == RECSDK_POOL_NONE ? max_D : (plan_only ? plan_total_D : grad_output.size(1)));
    b.max_D = static_cast<int32_t>(max_D);
    b.pooling_mode = static_cast<int32_t>(pooling_mode);
    b.optimizer = o.optimizer;
    b.total_hash_size_bits = static_cast<int32_t>(total_hash_size_bits);
    b.reduce_chunk = 64;
    b.learning_rate = static_cast<float>(o.lr);
    b.eps = static_cast<float>(o.eps);
    b.beta1 = static_cast<float>(o.beta1);
    b.beta2 = static_cast<float>(o.beta2);
    b.iter = o.iter;
    if (!ws.defined())
        ws = cached_workspace(table_set_cache(dev_weights),
                              static_cast<int64_t>(recsdk_tbe_backward_workspace_bytes(b.N, b.max_D)), dev_weights);
    b.workspace = ws.data_ptr();
    b.workspace_bytes = static_cast<size_t>(ws.numel());
    check_rc(recsdk_tbe_backward(&b, stream ? stream : cur_stream()), "split_embedding_backward_codegen_unweighted_exact_cuda");
    return Tensor();  // like the reference: state is updated in place, no weight gradient is returned
}

Tensor backward_adagrad_cuda(const Tensor& grad_output, const Tensor& dev_weights, const Tensor&, const Tensor&,
                             const Tensor&, const Tensor& weights_offsets, const Tensor& D_offsets, c10::SymInt max_D,
                             const Tensor& hash_size_cumsum, int64_t total_hash_size_bits, const Tensor& indices,
                             const Tensor& offsets, int64_t pooling_mode, const Tensor&, int64_t, int64_t, bool, int64_t,
                             int64_t, bool, bool, Tensor momentum1_dev, Tensor, Tensor, Tensor, const Tensor& hash_indices,
                             const Tensor& unique_ids, const Tensor& unique_offsets, const Tensor& unique_inverse,
                             const Tensor&, double eps, double learning_rate)
{
    OptArgs o{RECSDK_OPT_ADAGRAD, eps, learning_rate};
    return backward_exact(grad_output, dev_weights, weights_offsets, D_offsets, max_D.guard_int(__FILE__, __LINE__),
                          hash_size_cumsum, total_hash_size_bits, indices, offsets, pooling_mode, momentum1_dev, Tensor(),
                          hash_indices, unique_ids, unique_offsets, unique_inverse, o);
}

Tensor backward_adam_cuda(const Tensor& grad_output, const Tensor& dev_weights, const Tensor&, const Tensor&, const Tensor&,
                          const Tensor& weights_offsets, const Tensor& D_offsets, c10::SymInt max_D,
                          const Tensor& hash_size_cumsum, int64_t total_hash_size_bits, const Tensor& indices,
                          const Tensor& offsets, int64_t pooling_mode, const Tensor&, int64_t, int64_t, bool, int64_t, int64_t,
                          bool, bool, Tensor momentum1_dev, Tensor, Tensor, Tensor, Tensor momentum2_dev, Tensor, Tensor, Tensor,
                          const Tensor& hash_indices, const Tensor& unique_ids, const Tensor& unique_offsets,
                          const Tensor& unique_inverse, const Tensor&, double eps, double learning_rate, double beta1,
                          double beta2, int64_t iter)
{
    OptArgs o{RECSDK_OPT_ADAM, eps, learning_rate, beta1, beta2, iter};
    return backward_exact(grad_output, dev_weights, weights_offsets, D_offsets, max_D.guard_int(__FILE__, __LINE__),
                          hash_size_cumsum, total_hash_size_bits, indices, offsets, pooling_mode, momentum1_dev,
                          momentum2_dev, hash_indices, unique_ids, unique_offsets, unique_inverse, o);
}

Tensor backward_sgd_cuda(const Tensor& grad_output, const Tensor& dev_weights, const Tensor&, const Tensor&, const Tensor&,
                         const Tensor& weights_offsets, const Tensor& D_offsets, c10::SymInt max_D,
                         const Tensor& hash_size_cumsum, int64_t total_hash_size_bits, const Tensor& indices,
                         const Tensor& offsets, int64_t pooling_mode, const Tensor&, int64_t, int64_t, bool, int64_t, int64_t,
                         bool, bool, const Tensor& hash_indices, const Tensor& unique_ids, const Tensor& unique_offsets,
                         const Tensor& unique_inverse, const Tensor&, double learning_rate)
{
    OptArgs o{RECSDK_OPT_SGD, 0.0, learning_rate};
    return backward_exact(grad_output, dev_weights, weights_offsets, D_offsets, max_D.guard_int(__FILE__, __LINE__),
                          hash_size_cumsum, total_hash_size_bits, indices, offsets, pooling_mode, Tensor(), Tensor(),
                          hash_indices, unique_ids, unique_offsets, unique_inverse, o);
}

// ---------------------------------------------------------------------------- autograd lookup functions
// Plan ahead (off by default; recsdk::set_plan_ahead(True)): the lookup functions enqueue the index work of their
// own backward on a high-priority side stream while the forward runs, and the backward only sums and updates.
// For the forward -> backward alternation of training.
static std::atomic<bool> g_plan_ahead{false};
void set_plan_ahead(bool on) { g_plan_ahead.store(on); }
bool get_plan_ahead() { return g_plan_ahead.load(); }

// One Function for the three optimizers (the reference has SplitLookupAdagrad / SplitLookupAdam / SplitLookupSgd,
// e.g. backward_codegen_adam_unweighted_exact.cpp:65-284): forward = pooled gather, backward = optional clamp of
// the incoming gradient + fused segment-sum / optimizer, no gradient for any input.
class SplitLookup : public torch::autograd::Function<SplitLookup> {
public:
    static variable_list forward(AutogradContext* ctx, const Tensor& placeholder_autograd_tensor, int64_t optimizer,
                                 const Tensor& dev_weights, const Tensor& weights_offsets, const Tensor& D_offsets,
                                 int64_t total_D, int64_t max_D, const Tensor& hash_size_cumsum,
                                 int64_t total_hash_size_bits, const Tensor& indices,
                                 const std::optional<Tensor>& hash_indices_, const std::optional<Tensor>& unique_ids_,
                                 const std::optional<Tensor>& unique_offsets_, const std::optional<Tensor>& unique_inverse_,
                                 const Tensor& offsets, int64_t pooling_mode, bool gradient_clipping, double max_gradient,
                                 const std::optional<Tensor>& momentum1_, const std::optional<Tensor>& momentum2_, double eps,
                                 double lr, double beta1, double beta2, int64_t iter)
    {
        if (weights_offsets.size(0) == 0) return {Tensor()};
        // optional tensors travel through apply() as std::optional (an undefined Tensor argument is rejected there)
        const Tensor hash_indices = hash_indices_.value_or(Tensor()), unique_ids = unique_ids_.value_or(Tensor()),
                     unique_offsets = unique_offsets_.value_or(Tensor()), unique_inverse = unique_inverse_.value_or(Tensor()),
                     momentum1 = momentum1_.value_or(Tensor()), momentum2 = momentum2_.value_or(Tensor());
        ctx->save_for_backward({dev_weights, weights_offsets, D_offsets, hash_size_cumsum, indices, offsets, momentum1,
                                momentum2, hash_indices, unique_ids, unique_offsets, unique_inverse});
        ctx->saved_data["optimizer"] = optimizer;
        ctx->saved_data["max_D"] = max_D;
        ctx->saved_data["bits"] = total_hash_size_bits;
        ctx->saved_data["pooling_mode"] = pooling_mode;
        ctx->saved_data["gradient_clipping"] = gradient_clipping;
        ctx->saved_data["max_gradient"] = max_gradient;
        ctx->saved_data["eps"] = eps;
        ctx->saved_data["lr"] = lr;
        ctx->saved_data["beta1"] = beta1;
        ctx->saved_data["beta2"] = beta2;
        ctx->saved_data["iter"] = iter;
        ctx->saved_data["planned"] = false;
        const Tensor& plan_idx = pick(indices, hash_indices);
        if (g_plan_ahead.load() && dev_weights.is_cuda() && plan_idx.numel() > 0) {
            const c10::cuda::OptionalCUDAGuard guard(device_of(dev_weights));
            TableSetCache& c = table_set_cache(dev_weights);
            if (!c.side) {
                c.side = at::cuda::getStreamFromPool(/*isHighPriority=*/true, dev_weights.device().index());
                c.ready = std::make_unique<at::cuda::CUDAEvent>();
                c.done = std::make_unique<at::cuda::CUDAEvent>();
            }
            Tensor ws = cached_workspace(
                c, static_cast<int64_t>(recsdk_tbe_backward_workspace_bytes(plan_idx.numel(), static_cast<int32_t>(max_D))),
                dev_weights);
            auto cur = at::cuda::getCurrentCUDAStream();
            c.ready->record(cur);
            c.ready->block(*c.side);  // the indices are complete (and the previous backward is done with the workspace)
            for (const Tensor* t : {&plan_idx, &offsets, &unique_ids, &unique_offsets, &unique_inverse})
                if (t->defined() && t->numel() > 0)
                    c10::cuda::CUDACachingAllocator::recordStream(t->storage().data_ptr(), *c.side);  // read on the side stream
            OptArgs o{static_cast<int>(optimizer), eps, lr, beta1, beta2, iter};
            backward_exact(Tensor(), dev_weights, weights_offsets, D_offsets, max_D, hash_size_cumsum, total_hash_size_bits,
                           indices, offsets, pooling_mode, momentum1, momentum2, hash_indices, unique_ids, unique_offsets,
                           unique_inverse, o, RECSDK_BWD_PLAN_ONLY, ws, total_D, c.side->stream());
            c.done->record(*c.side);
            ctx->saved_data["planned"] = true;
        }
        const Tensor none;
        t_forward_leave_room = ctx->saved_data["planned"].toBool();
        Tensor out = forward_unweighted_cuda(dev_weights, none, none, none, weights_offsets, D_offsets, total_D, max_D,
                                             indices, offsets, pooling_mode, none, none, 0, false, hash_indices, none);
        t_forward_leave_room = false;
        return {out};
    }

    static variable_list backward(AutogradContext* ctx, variable_list grad_outputs)
    {
        const auto s = ctx->get_saved_variables();
        TORCH_CHECK_EQ(grad_outputs.size(), 1);
        Tensor g = grad_outputs[0];
        if (ctx->saved_data["gradient_clipping"].toBool()) {
            const double mg = ctx->saved_data["max_gradient"].toDouble();
            g = at::clamp(g, -mg, mg);  // backward_codegen_adagrad_unweighted_exact.cpp:153
        }
        OptArgs o{static_cast<int>(ctx->saved_data["optimizer"].toInt()), ctx->saved_data["eps"].toDouble(),
                  ctx->saved_data["lr"].toDouble(), ctx->saved_data["beta1"].toDouble(),
                  ctx->saved_data["beta2"].toDouble(), ctx->saved_data["iter"].toInt()};
        int flags = 0;
        Tensor ws;
        if (ctx->saved_data["planned"].toBool()) {
            // the plan (recorded on the side stream by the forward) is ordered before the apply phase
            const c10::cuda::OptionalCUDAGuard guard(device_of(s[0]));
            TableSetCache& c = table_set_cache(s[0]);
            c.done->block(at::cuda::getCurrentCUDAStream());
            flags = RECSDK_BWD_APPLY_ONLY;
            ws = c.ws;
        }
        backward_exact(g, s[0], s[1], s[2], ctx->saved_data["max_D"].toInt(), s[3], ctx->saved_data["bits"].toInt(), s[4],
                       s[5], ctx->saved_data["pooling_mode"].toInt(), s[6], s[7], s[8], s[9], s[10], s[11], o, flags, ws);
        return variable_list(25);  // no gradient for any of the 25 forward inputs
    }
};

static std::optional<Tensor> opt_or_empty(const std::optional<Tensor>& t)
{
    return (t.has_value() && t->defined()) ? t : std::nullopt;
}

Tensor lookup_adagrad_function(
    const Tensor& placeholder_autograd_tensor, const Tensor& dev_weights, const Tensor&, const Tensor&, const Tensor&,
    const Tensor& weights_offsets, const Tensor& D_offsets, c10::SymInt total_D, c10::SymInt max_D,
    const Tensor& hash_size_cumsum, int64_t total_hash_size_bits, const Tensor& indices, const Tensor& offsets,
    int64_t pooling_mode, const std::optional<Tensor>& indice_weights, const std::optional<Tensor>&, const Tensor&,
    bool gradient_clipping, double max_gradient, bool, Tensor momentum1_dev, Tensor, Tensor, Tensor,
    const std::optional<Tensor>& hash_indices, const std::optional<Tensor>& unique_ids,
    const std::optional<Tensor>& unique_offsets, const std::optional<Tensor>& unique_inverse, double eps,
    double learning_rate, int64_t, const std::optional<Tensor>&, const std::optional<Tensor>&,
    const std::optional<Tensor>&, c10::SymInt, c10::SymInt, c10::SymInt, bool, bool, bool, const std::optional<Tensor>&,
    const std::optional<Tensor>&, int64_t, bool, double)
{
    TORCH_CHECK(!indice_weights.has_value(), "weighted lookups are not supported");
    return SplitLookup::apply(placeholder_autograd_tensor, RECSDK_OPT_ADAGRAD, dev_weights, weights_offsets, D_offsets,
                              total_D.guard_int(__FILE__, __LINE__), max_D.guard_int(__FILE__, __LINE__), hash_size_cumsum,
                              total_hash_size_bits, indices, opt_or_empty(hash_indices), opt_or_empty(unique_ids),
                              opt_or_empty(unique_offsets), opt_or_empty(unique_inverse), offsets, pooling_mode,
                              gradient_clipping, max_gradient, std::optional<Tensor>(momentum1_dev), std::nullopt, eps,
                              learning_rate, 0.0, 0.0, 0)[0];
}

Tensor lookup_adam_function(
    const Tensor& placeholder_autograd_tensor, const Tensor& dev_weights, const Tensor&, const Tensor&, const Tensor&,
    const Tensor& weights_offsets, const Tensor& D_offsets, c10::SymInt total_D, c10::SymInt max_D,
    const Tensor& hash_size_cumsum, int64_t total_hash_size_bits, const Tensor& indices, const Tensor& offsets,
    int64_t pooling_mode, const std::optional<Tensor>& indice_weights, const std::optional<Tensor>&, const Tensor&,
    bool gradient_clipping, double max_gradient, bool, Tensor momentum1_dev, Tensor, Tensor, Tensor, Tensor momentum2_dev,
    Tensor, Tensor, Tensor, const std::optional<Tensor>& hash_indices, const std::optional<Tensor>& unique_ids,
    const std::optional<Tensor>& unique_offsets, const std::optional<Tensor>& unique_inverse, double eps,
    double learning_rate, double beta1, double beta2, double, int64_t iter, int64_t, const std::optional<Tensor>&,
    const std::optional<Tensor>&, const std::optional<Tensor>&, c10::SymInt, c10::SymInt, c10::SymInt, bool, bool, bool,
    const std::optional<Tensor>&, const std::optional<Tensor>&, bool, double)
{
    TORCH_CHECK(!indice_weights.has_value(), "weighted lookups are not supported");
    return SplitLookup::apply(placeholder_autograd_tensor, RECSDK_OPT_ADAM, dev_weights, weights_offsets, D_offsets,
                              total_D.guard_int(__FILE__, __LINE__), max_D.guard_int(__FILE__, __LINE__), hash_size_cumsum,
                              total_hash_size_bits, indices, opt_or_empty(hash_indices), opt_or_empty(unique_ids),
                              opt_or_empty(unique_offsets), opt_or_empty(unique_inverse), offsets, pooling_mode,
                              gradient_clipping, max_gradient, std::optional<Tensor>(momentum1_dev),
                              std::optional<Tensor>(momentum2_dev), eps, learning_rate, beta1, beta2, iter)[0];
}

Tensor lookup_sgd_function(
    const Tensor& placeholder_autograd_tensor, const Tensor& dev_weights, const Tensor&, const Tensor&, const Tensor&,
    const Tensor& weights_offsets, const Tensor& D_offsets, c10::SymInt total_D, c10::SymInt max_D,
    const Tensor& hash_size_cumsum, int64_t total_hash_size_bits, const Tensor& indices, const Tensor& offsets,
    int64_t pooling_mode, const std::optional<Tensor>& indice_weights, const std::optional<Tensor>&, const Tensor&,
    bool gradient_clipping, double max_gradient, bool, const std::optional<Tensor>& hash_indices,
    const std::optional<Tensor>& unique_ids, const std::optional<Tensor>& unique_offsets,
    const std::optional<Tensor>& unique_inverse, double learning_rate, int64_t, const std::optional<Tensor>&,
    const std::optional<Tensor>&, const std::optional<Tensor>&, c10::SymInt, c10::SymInt, c10::SymInt, bool, bool, bool,
    const std::optional<Tensor>&, const std::optional<Tensor>&, int64_t, bool, double)
{
    TORCH_CHECK(!indice_weights.has_value(), "weighted lookups are not supported");
    return SplitLookup::apply(placeholder_autograd_tensor, RECSDK_OPT_SGD, dev_weights, weights_offsets, D_offsets,
                              total_D.guard_int(__FILE__, __LINE__), max_D.guard_int(__FILE__, __LINE__), hash_size_cumsum,
                              total_hash_size_bits, indices, opt_or_empty(hash_indices), opt_or_empty(unique_ids),
                              opt_or_empty(unique_offsets), opt_or_empty(unique_inverse), offsets, pooling_mode,
                              gradient_clipping, max_gradient, std::nullopt, std::nullopt, 0.0, learning_rate, 0.0, 0.0, 0)[0];
}

// ---------------------------------------------------------------------------- schemas
static const char* kFwdSchema =
    "split_embedding_codegen_forward_unweighted_cuda(Tensor dev_weights, Tensor uvm_weights, Tensor lxu_cache_weights, "
    "Tensor weights_placements, Tensor weights_offsets, Tensor D_offsets, SymInt total_D, SymInt max_D, Tensor indices, "
    "Tensor offsets, int pooling_mode, Tensor lxu_cache_locations, Tensor uvm_cache_stats, int output_dtype, "
    "bool is_experimental, Tensor hash_indices = None, Tensor offset_per_key = None) -> Tensor";

#define RECSDK_LOOKUP_HEAD                                                                                             \
    "Tensor placeholder_autograd_tensor, Tensor(a!) dev_weights, Tensor(b!) uvm_weights, Tensor lxu_cache_weights, "   \
    "Tensor weights_placements, Tensor weights_offsets, Tensor D_offsets, SymInt total_D, SymInt max_D, "              \
    "Tensor hash_size_cumsum, int total_hash_size_bits, Tensor indices, Tensor offsets, int pooling_mode, "            \
    "Tensor? indice_weights, Tensor? feature_requires_grad, Tensor lxu_cache_locations, bool gradient_clipping, "      \
    "float max_gradient, bool stochastic_rounding, "
#define RECSDK_LOOKUP_UNIQ \
    "Tensor? hash_indices = None, Tensor? unique_ids = None, Tensor? unique_offsets = None, Tensor? unique_inverse = None, "
#define RECSDK_LOOKUP_VBE                                                                                              \
    "int output_dtype=0, Tensor? B_offsets=None, Tensor? vbe_output_offsets_feature_rank=None, "                       \
    "Tensor? vbe_B_offsets_rank_per_feature=None, SymInt max_B=-1, SymInt max_B_feature_rank=-1, "                     \
    "SymInt vbe_output_size=-1, bool is_experimental=False, bool use_uniq_cache_locations_bwd=False, "                 \
    "bool use_homogeneous_placements=False, Tensor? uvm_cache_stats=None, Tensor? prev_iter_dev=None, "
#define RECSDK_MOM1 "Tensor momentum1_dev, Tensor momentum1_uvm, Tensor momentum1_placements, Tensor momentum1_offsets, "
#define RECSDK_MOM2 "Tensor momentum2_dev, Tensor momentum2_uvm, Tensor momentum2_placements, Tensor momentum2_offsets, "
#define RECSDK_BWD_HEAD                                                                                                \
    "Tensor grad_output, Tensor(a!) dev_weights, Tensor(b!) uvm_weights, Tensor lxu_cache_weights, "                   \
    "Tensor weights_placements, Tensor weights_offsets, Tensor D_offsets, SymInt max_D, Tensor hash_size_cumsum, "     \
    "int total_hash_size_bits, Tensor indices, Tensor offsets, int pooling_mode, Tensor lxu_cache_locations, "         \
    "int unused_, int max_segment_length_per_warp, bool stochastic_rounding, int info_B_num_bits, "                    \
    "int info_B_mask_int64, bool use_uniq_cache_locations, bool use_homogeneous_placements, "
#define RECSDK_BWD_UNIQ                                                                                                \
    "Tensor hash_indices = None, Tensor unique_ids = None, Tensor unique_offsets = None, Tensor unique_inverse = None, " \
    "Tensor offset_per_key = None, "

static void define_and_implement(torch::Library& m)
{
    m.def(kFwdSchema);
    m.def("split_embedding_codegen_lookup_adagrad_function(" RECSDK_LOOKUP_HEAD RECSDK_MOM1 RECSDK_LOOKUP_UNIQ
          "float eps = 0, float learning_rate = 0, " RECSDK_LOOKUP_VBE
          "int iter=0, bool apply_global_weight_decay=False, float gwd_lower_bound=0) -> Tensor");
    m.def("split_embedding_codegen_lookup_adam_function(" RECSDK_LOOKUP_HEAD RECSDK_MOM1 RECSDK_MOM2 RECSDK_LOOKUP_UNIQ
          "float eps = 0, float learning_rate = 0, float beta1 = 0, float beta2 = 0, float weight_decay = 0, int iter = 0, "
          RECSDK_LOOKUP_VBE "bool apply_global_weight_decay=False, float gwd_lower_bound=0) -> Tensor");
    m.def("split_embedding_codegen_lookup_sgd_function(" RECSDK_LOOKUP_HEAD RECSDK_LOOKUP_UNIQ "float learning_rate = 0, "
          RECSDK_LOOKUP_VBE "int iter=0, bool apply_global_weight_decay=False, float gwd_lower_bound=0) -> Tensor");
    m.def("split_embedding_backward_codegen_adagrad_unweighted_exact_cuda(" RECSDK_BWD_HEAD RECSDK_MOM1 RECSDK_BWD_UNIQ
          "float eps = 0, float learning_rate = 0) -> Tensor");
    m.def("split_embedding_backward_codegen_adam_unweighted_exact_cuda(" RECSDK_BWD_HEAD RECSDK_MOM1 RECSDK_MOM2 RECSDK_BWD_UNIQ
          "float eps = 0, float learning_rate = 0, float beta1 = 0, float beta2 = 0, int iter = 0) -> Tensor");
    m.def("split_embedding_backward_codegen_sgd_unweighted_exact_cuda(" RECSDK_BWD_HEAD RECSDK_BWD_UNIQ
          "float learning_rate = 0) -> Tensor");

    const auto cuda = c10::DispatchKey::CUDA;
    const auto autograd = c10::DispatchKey::Autograd;
    m.impl("split_embedding_codegen_forward_unweighted_cuda", torch::dispatch(cuda, TORCH_FN(forward_unweighted_cuda)));
    m.impl("split_embedding_backward_codegen_adagrad_unweighted_exact_cuda", torch::dispatch(cuda, TORCH_FN(backward_adagrad_cuda)));
    m.impl("split_embedding_backward_codegen_adam_unweighted_exact_cuda", torch::dispatch(cuda, TORCH_FN(backward_adam_cuda)));
    m.impl("split_embedding_backward_codegen_sgd_unweighted_exact_cuda", torch::dispatch(cuda, TORCH_FN(backward_sgd_cuda)));
    m.impl("split_embedding_codegen_lookup_adagrad_function", torch::dispatch(autograd, TORCH_FN(lookup_adagrad_function)));
    m.impl("split_embedding_codegen_lookup_adam_function", torch::dispatch(autograd, TORCH_FN(lookup_adam_function)));
    m.impl("split_embedding_codegen_lookup_sgd_function", torch::dispatch(autograd, TORCH_FN(lookup_sgd_function)));
}

// ---------------------------------------------------------------------------- IdsMapper / bucketize
static void raise_on_status(const Tensor& status, const char* where)
{
    const Tensor h = status.cpu();  // synchronises, like the reference's TORCH_CHECK inside its host loop
    const int64_t* s = h.data_ptr<int64_t>();
    if (s[0] == 0) return;
    const int code = static_cast<int>(s[0]);
    const int64_t d0 = s[1];
    status.zero_();
    if (code == RECSDK_ERR_NEGATIVE_KEY) TORCH_CHECK(false, where, ":  Invalid key value: ", d0);
    if (code == RECSDK_ERR_TABLE_FULL)
        TORCH_CHECK(false, where, ": Ids map reached maxIndex = ", d0, " please reallocate a larger buffer.");
    TORCH_CHECK(false, where, ": ", recsdk_error_string(code));
}

// NS tags the registration namespace (a C++ type can back only one registered class): 0 = recsdk::, 1 = hybrid::
template <int NS>
class IdsMapperT : public torch::CustomClassHolder {
public:
    IdsMapperT(int64_t initMaxIndex, bool onlyDeviceMem) : initMaxIndex_(initMaxIndex)
    {
        TORCH_CHECK(initMaxIndex > 0, "initMaxIndex must be positive");
        const auto dev = at::Device(at::kCUDA, at::cuda::current_device());
        const auto i64 = at::TensorOptions().dtype(at::kLong).device(dev);
        int64_t cap = 16;
        while (cap < 2 * initMaxIndex + 1) cap <<= 1;
        table_ = at::empty({cap * 2}, i64);
        slot_key_ = at::empty({initMaxIndex}, i64);
        mark_ = at::empty({initMaxIndex}, i64.dtype(at::kInt));
        counters_ = at::zeros({4}, i64);
        status_ = at::zeros({RECSDK_STATUS_WORDS}, i64);
        m_ = recsdk_mapper_t{table_.data_ptr<int64_t>(), cap, slot_key_.data_ptr<int64_t>(), mark_.data_ptr<int32_t>(),
                             counters_.data_ptr<int64_t>(), initMaxIndex, onlyDeviceMem ? 1 : 0};
        check_rc(recsdk_mapper_init(&m_, cur_stream()), "IdsMapper");
    }

    std::tuple<Tensor, Tensor, Tensor> UniqueAndLookup(const Tensor& globalIds)
    {
        TORCH_CHECK(globalIds.is_cuda(), "globalIds must be on the GPU but on ", globalIds.device());
        TORCH_CHECK(globalIds.scalar_type() == at::kLong,
                    "globalIds must be int64_t tensor expected but got a tensor with dtype: ", globalIds.scalar_type());
        const Tensor ids = globalIds.contiguous();
        const int64_t n = ids.numel();
        Tensor hi = at::empty_like(ids), uq = at::empty({std::max<int64_t>(n, 1)}, ids.options()),
               inv = at::empty({std::max<int64_t>(n, 1)}, ids.options()), cnt = at::zeros({1}, ids.options());
        Tensor ws = workspace(n);
        check_rc(recsdk_mapper_ids2indices_unique(&m_, ids.data_ptr<int64_t>(), n, hi.data_ptr<int64_t>(),
                                                  uq.data_ptr<int64_t>(), inv.data_ptr<int64_t>(), cnt.data_ptr<int64_t>(),
                                                  status_.data_ptr<int64_t>(), ws.data_ptr(), ws.numel(), cur_stream()),
                 "ids2indices_unique");
        raise_on_status(status_, "ids2indices_unique");
        const int64_t u = cnt.item<int64_t>();
        return {hi, uq.narrow(0, 0, u), inv.narrow(0, 0, n)};
    }

    void UniqueAndLookupOut(const Tensor& globalIds, const Tensor& hashIndices, const Tensor& offset, const Tensor& unique,
                            const Tensor& uniqueIds, const Tensor& uniqueInverse, const Tensor& uniqueOffset, int64_t tableId)
    {
        enqueue_out(globalIds, hashIndices, offset, unique, uniqueIds, uniqueInverse, uniqueOffset, tableId);
        raise_on_status(status_, "ids2indices_unique_out");
    }

    static void ParallelUniqueHashOut(const c10::List<c10::intrusive_ptr<IdsMapperT>>& mappers, const Tensor& globalIds,
                                      const Tensor& hashIndices, const Tensor& offsets, const Tensor& unique,
                                      const Tensor& uniqueIds, const Tensor& uniqueInverse, const Tensor& uniqueOffset)
    {
        for (size_t t = 0; t < mappers.size(); ++t) {
            const c10::intrusive_ptr<IdsMapperT> m = mappers.get(t);
            m->enqueue_out(globalIds, hashIndices, offsets, unique, uniqueIds, uniqueInverse, uniqueOffset,
                           static_cast<int64_t>(t));
        }
        for (size_t t = 0; t < mappers.size(); ++t) {
            const c10::intrusive_ptr<IdsMapperT> m = mappers.get(t);
            raise_on_status(m->status_, "parallel_ids2indices_unique_out");
        }
    }

    int64_t size() { return counters_.cpu().data_ptr<int64_t>()[0]; }

private:
    Tensor workspace(int64_t n)
    {
        const int64_t need = static_cast<int64_t>(recsdk_mapper_workspace_bytes(n));
        if (!ws_.defined() || ws_.numel() < need) ws_ = at::empty({need}, table_.options().dtype(at::kByte));
        return ws_;
    }
    void enqueue_out(const Tensor& globalIds, const Tensor& hashIndices, const Tensor& offset, const Tensor& unique,
                     const Tensor& uniqueIds, const Tensor& uniqueInverse, const Tensor& uniqueOffset, int64_t tableId)
    {
        check_i64(globalIds, "globalIds");
        check_i64(hashIndices, "hashIndices");
        check_i64(unique, "unique");
        check_i64(uniqueIds, "uniqueIds");
        check_i64(uniqueInverse, "uniqueInverse");
        check_i64(uniqueOffset, "uniqueOffset");
        TORCH_CHECK(offset.numel() - 1 > tableId, "offset must be equal to table size + 1");
        const Tensor off = offset.cpu();  // segment bounds are host scalars for the launch
        const int64_t start = off.data_ptr<int64_t>()[tableId], end = off.data_ptr<int64_t>()[tableId + 1];
        Tensor ws = workspace(end - start);
        check_rc(recsdk_mapper_unique_out(&m_, globalIds.data_ptr<int64_t>(), hashIndices.data_ptr<int64_t>(), start,
                                          end - start, unique.data_ptr<int64_t>(), uniqueIds.data_ptr<int64_t>(),
                                          uniqueInverse.data_ptr<int64_t>(), uniqueOffset.data_ptr<int64_t>(), tableId,
                                          status_.data_ptr<int64_t>(), ws.data_ptr(), ws.numel(), cur_stream()),
                 "ids2indices_unique_out");
    }

    int64_t initMaxIndex_;
    Tensor table_, slot_key_, mark_, counters_, status_, ws_;
    recsdk_mapper_t m_;
};
using IdsMapper = IdsMapperT<0>;
using HybridIdsMapper = IdsMapperT<1>;

// (new_lengths, new_indices, None, None, unbucketize_permute, None, ids_counts), bucketize.cpp:214-282
std::tuple<Tensor, Tensor, std::optional<Tensor>, std::optional<Tensor>, std::optional<Tensor>, std::optional<Tensor>, Tensor>
block_bucketize_sparse_features(const Tensor& lengths, const Tensor& indices, bool bucketize_pos, bool sequence,
                                const Tensor& block_sizes, int64_t bucket_size, const std::optional<Tensor>& total_num_blocks,
                                const std::optional<Tensor>& weights, const std::optional<Tensor>& batch_size_per_feature,
                                int64_t max_B, const std::optional<std::vector<Tensor>>& block_bucketize_pos,
                                bool return_bucket_mapping, bool keep_orig_idx, bool do_unique, bool return_count)
{
    TORCH_CHECK(lengths.defined() && lengths.numel() > 0, "Lengths tensor is an empty tensor");
    TORCH_CHECK(indices.defined() && indices.numel() > 0, "Indices tensor is an empty tensor");
    TORCH_CHECK(!weights.has_value(), "Weighted KJT is currently not supported");
    TORCH_CHECK(!bucketize_pos, "Bucket position tracking is not implemented");
    TORCH_CHECK(!return_bucket_mapping, "Bucket mapping return is not supported");
    TORCH_CHECK(!batch_size_per_feature, "batchSize PerFeature return is not supported");
    TORCH_CHECK(!block_bucketize_pos, "block BucketizePos return is not supported");
    TORCH_CHECK(bucket_size > 0, "Bucket size must be greater than 0");
    check_i64(lengths, "lengths");
    check_i64(indices, "indices");
    const c10::cuda::OptionalCUDAGuard guard(device_of(indices));
    const int64_t n = indices.numel(), L = lengths.numel(), F = block_sizes.numel();
    TORCH_CHECK(F > 0, "blockSizes must have at least one element");
    const bool uniq = sequence && do_unique;
    Tensor new_lengths = at::empty({L * bucket_size}, lengths.options());
    Tensor new_indices = at::empty_like(indices), perm = at::empty_like(indices);
    Tensor counts = (uniq && return_count) ? at::empty_like(indices) : at::empty({0}, indices.options());
    Tensor num_out = at::zeros({1}, indices.options());
    Tensor ws = at::empty({static_cast<int64_t>(recsdk_bucketize_workspace_bytes(n, L, bucket_size))},
                          indices.options().dtype(at::kByte));
    check_rc(recsdk_bucketize(lengths.data_ptr<int64_t>(), L, indices.data_ptr<int64_t>(), n, F, bucket_size, uniq ? 1 : 0,
                              (uniq && return_count) ? 1 : 0, new_lengths.data_ptr<int64_t>(), new_indices.data_ptr<int64_t>(),
                              perm.data_ptr<int64_t>(), counts.numel() ? counts.data_ptr<int64_t>() : nullptr,
                              num_out.data_ptr<int64_t>(), ws.data_ptr(), ws.numel(), cur_stream()),
             "block_bucketize_sparse_features");
    if (uniq) {
        const int64_t k = num_out.item<int64_t>();  // the reference resize_()s to the unique count
        new_indices = new_indices.narrow(0, 0, k);
        if (return_count) counts = counts.narrow(0, 0, k);
    }
    return {new_lengths, new_indices, std::nullopt, std::nullopt, perm, std::nullopt, counts};
}

// ---------------------------------------------------------------------------- jagged-batch utilities
// permute2d_sparse_data.cpp:21-48, permute1d_sparse_data.cpp:57-93, asynchronous_complete_cumsum.cpp:18-25,
// jagged_to_padded_dense.cpp, dense_to_jagged.cpp of cust_op/framework/torch_plugin/torch_library/2.6.0
static std::tuple<Tensor, Tensor, std::optional<Tensor>> permute_sparse_impl(const Tensor& permute, const Tensor& lengths2d,
                                                                             const Tensor& values,
                                                                             const std::optional<Tensor>& weights,
                                                                             const std::optional<c10::SymInt>& sum)
{
    TORCH_CHECK(values.is_cuda(), "values must be a CUDA tensor");
    const c10::cuda::OptionalCUDAGuard guard(device_of(values));
    const Tensor perm = permute.to(at::kLong).contiguous();
    const Tensor len = lengths2d.to(at::kLong).contiguous();
    const Tensor vals = values.contiguous();
    TORCH_CHECK(vals.element_size() == 4 || vals.element_size() == 8, "values must have 4- or 8-byte elements");
    const int64_t T_in = len.size(0), B = len.size(1), T_out = perm.numel();
    Tensor w;
    if (weights.has_value() && weights->defined()) {
        TORCH_CHECK(weights->numel() == vals.numel(), "weights and values length mismatch: ", weights->numel(), " vs ",
                    vals.numel());
        w = weights->to(at::kFloat).contiguous();
    }
    int64_t total;
    if (sum.has_value() && sum->guard_int(__FILE__, __LINE__) > 0)
        total = sum->guard_int(__FILE__, __LINE__);
    else
        total = (T_out && B) ? len.index_select(0, perm).sum().item<int64_t>() : 0;
    Tensor out_len = at::empty({T_out, B}, len.options());
    Tensor out_vals = at::empty({total}, vals.options());
    Tensor out_w = w.defined() ? at::empty({total}, w.options()) : Tensor();
    Tensor status = at::zeros({RECSDK_STATUS_WORDS}, len.options());
    Tensor ws = at::empty({static_cast<int64_t>(recsdk_permute_sparse_workspace_bytes(T_in, T_out))},
                          len.options().dtype(at::kByte));
    check_rc(recsdk_permute_2d_sparse_data(perm.data_ptr<int64_t>(), T_out, len.data_ptr<int64_t>(), T_in, B, vals.data_ptr(),
                                           static_cast<int32_t>(vals.element_size()),
                                           w.defined() ? w.data_ptr<float>() : nullptr, out_len.data_ptr<int64_t>(),
                                           out_vals.data_ptr(), out_w.defined() ? out_w.data_ptr<float>() : nullptr, total,
                                           nullptr, status.data_ptr<int64_t>(), ws.data_ptr(), ws.numel(), cur_stream()),
             "permute_sparse_data");
    const Tensor st = status.cpu();
    TORCH_CHECK(st.data_ptr<int64_t>()[0] == 0, "permute_sparse_data: ", recsdk_error_string(static_cast<int>(st.data_ptr<int64_t>()[0])));
    std::optional<Tensor> ow;
    if (out_w.defined()) ow = out_w;
    return {out_len.to(lengths2d.scalar_type()), out_vals, ow};
}

std::tuple<Tensor, Tensor, std::optional<Tensor>> permute_2D_sparse_data(const Tensor& permute, const Tensor& lengths,
                                                                         const Tensor& values,
                                                                         const std::optional<Tensor>& weights,
                                                                         std::optional<c10::SymInt> permuted_lengths_sum)
{
    TORCH_CHECK(lengths.dim() == 2, "lengths must be 2-D");
    return permute_sparse_impl(permute, lengths, values, weights, permuted_lengths_sum);
}

std::tuple<Tensor, Tensor, std::optional<Tensor>> permute_1D_sparse_data(const Tensor& permute, const Tensor& lengths,
                                                                         const Tensor& values,
                                                                         const std::optional<Tensor>& weights,
                                                                         std::optional<c10::SymInt> permuted_lengths_sum)
{
    TORCH_CHECK(permute.dim() == 1 && lengths.dim() == 1 && values.dim() == 1, "permute, lengths and values must be 1-D");
    auto r = permute_sparse_impl(permute, lengths.view({-1, 1}), values, weights, permuted_lengths_sum);
    return {std::get<0>(r).view({-1}), std::get<1>(r), std::get<2>(r)};
}

Tensor asynchronous_complete_cumsum(const Tensor& offset)
{
    TORCH_CHECK(offset.is_cuda(), "offset must be a CUDA tensor");
    const c10::cuda::OptionalCUDAGuard guard(device_of(offset));
    const Tensor x = offset.to(at::kLong).contiguous();
    const int64_t n = x.numel();
    Tensor out = at::empty({n + 1}, x.options());
    Tensor ws = at::empty({static_cast<int64_t>(recsdk_complete_cumsum_workspace_bytes(n))}, x.options().dtype(at::kByte));
    check_rc(recsdk_complete_cumsum(x.data_ptr<int64_t>(), n, out.data_ptr<int64_t>(), ws.data_ptr(), ws.numel(), cur_stream()),
             "asynchronous_complete_cumsum");
    return out.to(offset.scalar_type());
}

static Tensor jagged_to_dense_impl(const Tensor& values, const std::vector<Tensor>& offsets, int64_t max_lengths,
                                   double padding_value)
{
    TORCH_CHECK(values.dim() == 2, "values must be 2-D");
    TORCH_CHECK(offsets.size() == 1, "offsets must contain exactly 1 tensor, but got ", offsets.size(), " tensors");
    TORCH_CHECK(max_lengths > 0, "max_lengths must be positive, but got ", max_lengths);
    TORCH_CHECK(values.is_cuda() && values.scalar_type() == at::kFloat, "values must be a CUDA fp32 tensor");
    const c10::cuda::OptionalCUDAGuard guard(device_of(values));
    const Tensor v = values.contiguous();
    const Tensor offs = offsets[0].to(at::kLong).contiguous();
    const int64_t B = offs.numel() - 1, D = v.size(1);
    Tensor out = at::empty({B, max_lengths, D}, v.options());
    check_rc(recsdk_jagged_to_padded_dense(v.data_ptr<float>(), offs.data_ptr<int64_t>(), B, static_cast<int32_t>(D),
                                           max_lengths, static_cast<float>(padding_value), out.data_ptr<float>(), cur_stream()),
             "jagged_to_padded_dense");
    return out;
}

static Tensor dense_to_jagged_impl(const Tensor& dense, const std::vector<Tensor>& offsets, int64_t total_L)
{
    TORCH_CHECK(dense.dim() == 3, "dense must be 3-D [B, L, D]");
    TORCH_CHECK(offsets.size() == 1, "offsets must contain exactly 1 tensor, but got ", offsets.size(), " tensors");
    TORCH_CHECK(dense.is_cuda() && dense.scalar_type() == at::kFloat, "dense must be a CUDA fp32 tensor");
    const c10::cuda::OptionalCUDAGuard guard(device_of(dense));
    const Tensor d = dense.contiguous();
    const Tensor offs = offsets[0].to(at::kLong).contiguous();
    const int64_t B = d.size(0), L = d.size(1), D = d.size(2);
    if (total_L < 0) total_L = offs[-1].item<int64_t>();
    Tensor values = at::empty({total_L, D}, d.options());
    check_rc(recsdk_dense_to_jagged(d.data_ptr<float>(), offs.data_ptr<int64_t>(), B, static_cast<int32_t>(D), L,
                                    values.data_ptr<float>(), cur_stream()),
             "dense_to_jagged");
    return values;
}

struct JaggedToPaddedDenseFn : public torch::autograd::Function<JaggedToPaddedDenseFn> {
    static Tensor forward(AutogradContext* ctx, const Tensor& values, const Tensor& offsets, int64_t max_lengths,
                          double padding_value)
    {
        at::AutoDispatchBelowADInplaceOrView guard;
        ctx->save_for_backward({offsets});
        ctx->saved_data["total_L"] = values.size(0);
        return jagged_to_dense_impl(values, {offsets}, max_lengths, padding_value);
    }
    static variable_list backward(AutogradContext* ctx, variable_list grads)
    {
        const Tensor offsets = ctx->get_saved_variables()[0];
        return {dense_to_jagged_impl(grads[0], {offsets}, ctx->saved_data["total_L"].toInt()), Tensor(), Tensor(), Tensor()};
    }
};

struct DenseToJaggedFn : public torch::autograd::Function<DenseToJaggedFn> {
    static Tensor forward(AutogradContext* ctx, const Tensor& dense, const Tensor& offsets, int64_t total_L)
    {
        at::AutoDispatchBelowADInplaceOrView guard;
        ctx->save_for_backward({offsets});
        ctx->saved_data["L"] = dense.size(1);
        return dense_to_jagged_impl(dense, {offsets}, total_L);
    }
    static variable_list backward(AutogradContext* ctx, variable_list grads)
    {
        const Tensor offsets = ctx->get_saved_variables()[0];
        return {jagged_to_dense_impl(grads[0], {offsets}, ctx->saved_data["L"].toInt(), 0.0), Tensor(), Tensor()};
    }
};

Tensor jagged_to_padded_dense_v1(const Tensor& values, std::vector<Tensor> offsets, int64_t max_lengths, double padding_value)
{
    TORCH_CHECK(offsets.size() == 1, "offsets must contain exactly 1 tensor, but got ", offsets.size(), " tensors");
    return JaggedToPaddedDenseFn::apply(values, offsets[0], max_lengths, padding_value);
}
Tensor jagged_to_padded_dense_v2(const Tensor& values, std::vector<Tensor> offsets, at::IntArrayRef max_lengths,
                                 double padding_value)
{
    TORCH_CHECK(max_lengths.size() == 1, "max_lengths must contain exactly one element, but got ", max_lengths.size());
    return jagged_to_padded_dense_v1(values, std::move(offsets), max_lengths[0], padding_value);
}
std::tuple<Tensor, std::vector<Tensor>> dense_to_jagged(const Tensor& dense, std::vector<Tensor> offsets,
                                                        std::optional<c10::SymInt> total_L)
{
    TORCH_CHECK(offsets.size() == 1, "offsets must contain exactly 1 tensor, but got ", offsets.size(), " tensors");
    const int64_t tl = total_L.has_value() ? total_L->guard_int(__FILE__, __LINE__) : -1;
    return {DenseToJaggedFn::apply(dense, offsets[0], tl), offsets};
}

// schema strings of the reference's TORCH_LIBRARY(mxrec) blocks, verbatim modulo whitespace
void define_and_implement_kjt(torch::Library& m)
{
    m.def("permute_2D_sparse_data(Tensor permute, Tensor lengths, Tensor values, Tensor? weights=None, "
          "SymInt? permuted_lengths_sum=None) -> (Tensor, Tensor, Tensor?)", &permute_2D_sparse_data);
    m.def("permute_1D_sparse_data(Tensor permute, Tensor lengths, Tensor values, Tensor? weights=None, "
          "SymInt? permuted_lengths_sum=None) -> (Tensor, Tensor, Tensor?)", &permute_1D_sparse_data);
    m.def("asynchronous_complete_cumsum(Tensor offset) -> Tensor", &asynchronous_complete_cumsum);
    m.def("jagged_to_padded_dense.v1(Tensor values, Tensor[] offsets, int max_lengths, float padding_value) -> Tensor",
          &jagged_to_padded_dense_v1);
    m.def("jagged_to_padded_dense.v2(Tensor values, Tensor[] offsets, int[] max_lengths, float padding_value) -> Tensor",
          &jagged_to_padded_dense_v2);
    m.def("dense_to_jagged(Tensor dense, Tensor[] offsets, SymInt? total_L=None) -> (Tensor, Tensor[])", &dense_to_jagged);
}

// ---------------------------------------------------------------------------- TF-flavour operators
// The four operators the reference registers with TensorFlow (cust_op/framework/tf_plugin/src/
// cust_embedding_by_address.cpp:19-52, lazy_adam.cpp:20-35, sgd.cpp:19-28), as torch operators with the same names,
// input order and attributes.  The TF ops return new tensors that alias their stateful inputs; here the state
// tensors are updated in place and returned.
Tensor embedding_lookup_by_address(const Tensor& address, int64_t embedding_dim, int64_t embedding_type)
{
    check_i64(address, "address");
    TORCH_CHECK(address.dim() == 1, "address must be a vector");
    TORCH_CHECK(embedding_type == 0, "only fp32 (embedding_type 0) is supported");
    TORCH_CHECK(embedding_dim > 0, "embedding_dim must be positive");
    Tensor out = at::empty({address.numel(), embedding_dim}, address.options().dtype(at::kFloat));
    check_rc(recsdk_lookup_by_address(address.data_ptr<int64_t>(), address.numel(), static_cast<int32_t>(embedding_dim),
                                      out.data_ptr<float>(), cur_stream()),
             "EmbeddingLookupByAddress");
    return out;
}

Tensor embedding_update_by_address(const Tensor& address, const Tensor& embedding, int64_t update_type)
{
    check_i64(address, "address");
    TORCH_CHECK(address.dim() == 1 && embedding.dim() == 2 && embedding.size(0) == address.numel(),
                "address [n] and embedding [n, dim] expected");
    TORCH_CHECK(embedding.is_cuda() && embedding.scalar_type() == at::kFloat && embedding.is_contiguous(),
                "embedding must be a contiguous float32 CUDA tensor");
    check_rc(recsdk_update_by_address(address.data_ptr<int64_t>(), address.numel(), static_cast<int32_t>(embedding.size(1)),
                                      embedding.data_ptr<float>(), static_cast<int32_t>(update_type), cur_stream()),
             "EmbeddingUpdateByAddress");
    return embedding;
}

static void check_f32(const Tensor& t, const char* name)
{
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous(), name,
                " must be a contiguous float32 CUDA tensor");
}

std::tuple<Tensor, Tensor, Tensor> lazy_adam(const Tensor& gradient, const Tensor& indices, Tensor input_m, Tensor input_v,
                                             Tensor input_var, const Tensor& lr, double beta1, double beta2,
                                             double epsilon)
{
    check_f32(gradient, "gradient");
    check_f32(input_m, "input_m");
    check_f32(input_v, "input_v");
    check_f32(input_var, "input_var");
    TORCH_CHECK(indices.is_cuda() && indices.scalar_type() == at::kInt && indices.is_contiguous(),
                "indices must be a contiguous int32 CUDA tensor");
    TORCH_CHECK(gradient.dim() == 2 && gradient.size(0) == indices.numel(), "gradient [n, dim] and indices [n] expected");
    TORCH_CHECK(input_m.numel() == input_var.numel() && input_v.numel() == input_var.numel(),
                "input_m / input_v / input_var must have the same size");
    const float lr_v = lr.item<float>();  // a scalar tensor in the reference's signature
    check_rc(recsdk_lazy_adam(gradient.data_ptr<float>(), indices.data_ptr<int32_t>(), indices.numel(),
                              static_cast<int32_t>(gradient.size(1)), input_m.data_ptr<float>(), input_v.data_ptr<float>(),
                              input_var.data_ptr<float>(), lr_v, static_cast<float>(beta1), static_cast<float>(beta2),
                              static_cast<float>(epsilon), cur_stream()),
             "LazyAdam");
    return {input_m, input_v, input_var};
}

Tensor sgd(const Tensor& gradient, const Tensor& indices, Tensor input_var, const Tensor& lr, double weightDecay)
{
    check_f32(gradient, "gradient");
    check_f32(input_var, "input_var");
    TORCH_CHECK(indices.is_cuda() && indices.is_contiguous() &&
                    (indices.scalar_type() == at::kInt || indices.scalar_type() == at::kLong),
                "indices must be a contiguous int32 or int64 CUDA tensor");
    TORCH_CHECK(gradient.dim() == 2 && gradient.size(0) == indices.numel(), "gradient [n, dim] and indices [n] expected");
    const Tensor idx64 = indices.scalar_type() == at::kLong ? indices : indices.to(at::kLong);
    const bool decay = weightDecay != 0.0;
    Tensor ws = decay ? at::empty({gradient.numel()}, gradient.options()) : Tensor();
    check_rc(recsdk_sgd(gradient.data_ptr<float>(), idx64.data_ptr<int64_t>(), idx64.numel(),
                        static_cast<int32_t>(gradient.size(1)), input_var.data_ptr<float>(), lr.item<float>(),
                        static_cast<float>(weightDecay), decay ? 1 : 0, decay ? ws.data_ptr() : nullptr,
                        decay ? static_cast<size_t>(ws.numel()) * 4 : 0, cur_stream()),
             "Sgd");
    return input_var;
}

void define_and_implement_tf_flavour(torch::Library& m)
{
    m.def("EmbeddingLookupByAddress(Tensor address, int embedding_dim, int embedding_type) -> Tensor",
          &embedding_lookup_by_address);
    m.def("EmbeddingUpdateByAddress(Tensor address, Tensor embedding, int update_type) -> Tensor",
          &embedding_update_by_address);
    m.def("LazyAdam(Tensor gradient, Tensor indices, Tensor(a!) input_m, Tensor(b!) input_v, Tensor(c!) input_var, Tensor lr, "
          "float beta1, float beta2, float epsilon) -> (Tensor(a!), Tensor(b!), Tensor(c!))", &lazy_adam);
    m.def("Sgd(Tensor gradient, Tensor indices, Tensor(a!) input_var, Tensor lr, float weightDecay=0.0) -> Tensor(a!)", &sgd);
}

}  // namespace recsdk_torch

#ifndef RECSDK_NO_FBGEMM_NS
TORCH_LIBRARY_FRAGMENT(fbgemm, m)
{
    recsdk_torch::define_and_implement(m);
    recsdk_torch::define_and_implement_kjt(m);
}
#endif

// the namespace the reference defines the jagged-batch utilities in
#ifndef RECSDK_NO_MXREC_NS
TORCH_LIBRARY(mxrec, m) { recsdk_torch::define_and_implement_kjt(m); }
#endif

TORCH_LIBRARY(recsdk, m)
{
    recsdk_torch::define_and_implement(m);
    m.class_<recsdk_torch::IdsMapper>("IdsMapper")
        .def(torch::init<int64_t, bool>())
        .def("ids2indices_unique", &recsdk_torch::IdsMapper::UniqueAndLookup)
        .def("ids2indices_unique_out", &recsdk_torch::IdsMapper::UniqueAndLookupOut)
        .def("size", &recsdk_torch::IdsMapper::size)
        .def_static("parallel_ids2indices_unique_out", &recsdk_torch::IdsMapper::ParallelUniqueHashOut);
    m.def("block_bucketize_sparse_features", &recsdk_torch::block_bucketize_sparse_features);
    m.def("set_plan_ahead(bool on) -> ()", &recsdk_torch::set_plan_ahead);
    m.def("get_plan_ahead() -> bool", &recsdk_torch::get_plan_ahead);
    recsdk_torch::define_and_implement_kjt(m);
    recsdk_torch::define_and_implement_tf_flavour(m);
}

// The reference's own registration names (hybrid_torchrec/src/bind_torch_lib.cpp:9-19): callers that say
// torch.classes.hybrid.IdsMapper / torch.ops.hybrid.block_bucketize_sparse_features_cpu keep working, with CUDA
// tensors.  Compile with -DRECSDK_NO_HYBRID_NS when the reference's libhybrid_cpp.so is loaded in the same process.
#ifndef RECSDK_NO_HYBRID_NS
TORCH_LIBRARY(hybrid, m)
{
    m.class_<recsdk_torch::HybridIdsMapper>("IdsMapper")
        .def(torch::init<int64_t, bool>())
        .def("ids2indices_unique", &recsdk_torch::HybridIdsMapper::UniqueAndLookup)
        .def("ids2indices_unique_out", &recsdk_torch::HybridIdsMapper::UniqueAndLookupOut)
        .def("size", &recsdk_torch::HybridIdsMapper::size)
        .def_static("parallel_ids2indices_unique_out", &recsdk_torch::HybridIdsMapper::ParallelUniqueHashOut);
    m.def("block_bucketize_sparse_features_cpu", &recsdk_torch::block_bucketize_sparse_features);
}
#endif
