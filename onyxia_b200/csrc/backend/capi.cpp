// extern "C" backend / session / tensor calls of onyxia_cuda.h.
#include <cstring>

#include "../ir/module_api.hpp"
#include "session.hpp"

using namespace ox;

#include "capi_types.hpp"

#define OX_TRY try {
#define OX_CATCH                                                                          \
    }                                                                                     \
    catch (const ox::Error& e) { return (ox_status)ox::set_error(e); }                    \
    catch (const std::exception& e) { return (ox_status)ox::set_error(ErrKind::Runtime, e.what()); }

extern "C" {

ox_status ox_backend_create_ex(const int32_t* device_ordinals, int32_t n_devices, const ox_backend_options* options,
                               ox_backend** out) {
    OX_TRY
    std::vector<int> devs;
    for (int i = 0; i < n_devices; i++) devs.push_back(device_ordinals[i]);
    oxrt::Options opt;
    if (options) {
        opt.without_fused = options->without_fused_kernels != 0;
        opt.disable_graphs = options->disable_graphs != 0;
        opt.disable_pattern_fusion = options->disable_pattern_fusion != 0;
        opt.disable_persist = options->disable_persistent_step != 0;
    }
    auto* b = new ox_backend();
    try {
        b->b = std::make_unique<oxrt::Backend>(devs, opt);
    } catch (...) {
        delete b;
        throw;
    }
    *out = b;
    return OX_OK;
    OX_CATCH
}

ox_status ox_backend_create(const int32_t* device_ordinals, int32_t n_devices, ox_backend** out) {
    return ox_backend_create_ex(device_ordinals, n_devices, nullptr, out);
}

ox_status ox_tp_unique_id(const char* nccl_library_path, uint8_t out[128]) {
    OX_TRY
    oxrt::tp_unique_id(nccl_library_path, out);
    return OX_OK;
    OX_CATCH
}

ox_status ox_backend_join_tp(ox_backend* b, int32_t rank, int32_t world, const uint8_t id[128], const char* nccl_library_path) {
    OX_TRY
    b->b->join(std::make_shared<oxrt::Communicator>(b->b->device(), rank, world, id, nccl_library_path));
    return OX_OK;
    OX_CATCH
}

int32_t ox_backend_peer_allreduce(const ox_backend* b) {
    const oxrt::Communicator* c = b->b->communicator();
    return c && c->peer_path_ready() ? 1 : 0;
}

void ox_backend_free(ox_backend* b) { delete b; }

int32_t ox_backend_supports(const ox_backend* b, const char* name) { return b->b->supports(name) ? 1 : 0; }

ox_status ox_backend_prepare(ox_backend* b, ox_module* module, ox_session** out) {
    std::unique_ptr<ox_module> owned(module);  // consumed, also on failure
    OX_TRY
    auto* s = new ox_session();
    try {
        s->s = b->b->prepare(std::move(owned->b.module()));
    } catch (...) {
        delete s;
        throw;
    }
    *out = s;
    return OX_OK;
    OX_CATCH
}

void ox_session_free(ox_session* s) { delete s; }

ox_status ox_session_upload(ox_session* s, int32_t dtype, const uint64_t* shape, int32_t rank, const void* bytes,
                            size_t nbytes, ox_tensor** out) {
    OX_TRY
    if (dtype < 0 || dtype >= kNumDTypes) fail(ErrKind::DType, "unknown dtype code");
    std::vector<int64_t> shp;
    for (int i = 0; i < rank; i++) shp.push_back((int64_t)shape[i]);
    auto* t = new ox_tensor();
    try {
        t->t = s->s->upload((DType)dtype, shp, bytes, nbytes);
    } catch (...) {
        delete t;
        throw;
    }
    *out = t;
    return OX_OK;
    OX_CATCH
}

ox_status ox_session_run(ox_session* s, const char* const* names, ox_tensor* const* inputs, int32_t n_in,
                         const char** out_names, ox_tensor** out_tensors, int32_t out_cap, int32_t* n_out) {
    OX_TRY
    std::vector<std::pair<std::string, oxrt::DTensor>> ins;
    for (int i = 0; i < n_in; i++) {
        if (!inputs[i]) fail(ErrKind::Binding, std::string("input '") + names[i] + "' is null");
        ins.emplace_back(names[i], inputs[i]->t);
    }
    auto outs = s->s->run(ins);
    if ((int)outs.size() > out_cap) fail(ErrKind::Runtime, "output array too small: module has " + std::to_string(outs.size()) + " outputs");
    const auto& names_store = s->s->output_names();
    for (size_t i = 0; i < outs.size(); i++) {
        out_names[i] = names_store[i].c_str();
        auto* t = new ox_tensor();
        t->t = std::move(outs[i].second);
        out_tensors[i] = t;
    }
    *n_out = (int32_t)outs.size();
    return OX_OK;
    OX_CATCH
}

int32_t ox_session_num_outputs(const ox_session* s) { return (int32_t)s->s->output_names().size(); }

ox_status ox_session_download(ox_session* s, const ox_tensor* t, void* dst, size_t cap, size_t* written) {
    OX_TRY
    s->s->download(t->t, dst, cap, written);
    return OX_OK;
    OX_CATCH
}

ox_tensor* ox_tensor_clone(const ox_tensor* t) { return t ? new ox_tensor(*t) : nullptr; }
void ox_tensor_release(ox_tensor* t) { delete t; }

ox_status ox_tensor_describe(const ox_tensor* t, int32_t* dtype, uint64_t* shape, int32_t shape_cap, int32_t* rank) {
    OX_TRY
    if (dtype) *dtype = (int32_t)t->t.dtype;
    if (rank) *rank = (int32_t)t->t.shape.size();
    if (shape) {
        if ((size_t)shape_cap < t->t.shape.size()) fail(ErrKind::Runtime, "shape array too small");
        for (size_t i = 0; i < t->t.shape.size(); i++) shape[i] = (uint64_t)t->t.shape[i];
    }
    return OX_OK;
    OX_CATCH
}

size_t ox_tensor_nbytes(const ox_tensor* t) { return t->t.nbytes(); }

ox_status ox_session_wait_idle(ox_session* s) {
    OX_TRY
    s->s->wait_idle();
    return OX_OK;
    OX_CATCH
}

uint64_t ox_session_resident_bytes(const ox_session* s) { return s->s->resident_bytes(); }
uint64_t ox_session_peak_resident_bytes(const ox_session* s) { return s->s->peak_resident_bytes(); }
void ox_session_pool_stats(const ox_session* s, uint64_t* fresh, uint64_t* reuses) {
    if (fresh) *fresh = s->s->pool().fresh_allocations;
    if (reuses) *reuses = s->s->pool().reuses;
}

int32_t ox_session_enable_profiling(ox_session* s, int32_t on) {
    s->s->profiling = on != 0;
    return 1;
}

int32_t ox_session_take_timings(ox_session* s, ox_kernel_timing* out, int32_t cap) {
    try {
        s->taken = s->s->take_timings();
    } catch (const std::exception&) {
        s->taken.clear();
    }
    int n = (int)s->taken.size();
    for (int i = 0; i < n && i < cap; i++) {
        out[i].kernel = s->taken[i].kernel.c_str();
        out[i].node = s->taken[i].node.c_str();
        out[i].time_ns = s->taken[i].time_ns;
    }
    return n;
}

ox_status ox_session_timer_start(ox_session* s) {
    OX_TRY
    s->s->timer_start();
    return OX_OK;
    OX_CATCH
}

ox_status ox_session_timer_stop(ox_session* s, float* elapsed_ms) {
    OX_TRY
    *elapsed_ms = s->s->timer_stop();
    return OX_OK;
    OX_CATCH
}

uint64_t ox_session_launch_count(const ox_session* s) { return s->s->launch_count; }

void ox_session_plan_stats(const ox_session* s, uint64_t out[9]) {
    out[5] = s->s->host_runs;
    for (int i = 0; i < 3; i++) out[6 + i] = (uint64_t)s->s->host_us[i];
    out[0] = s->s->plans_built;
    out[1] = s->s->plans_updated;
    out[2] = s->s->plans_reused;
    out[3] = s->s->graph_launches;
    out[4] = s->s->graph_node_updates;
}

ox_status ox_session_argmax_last(ox_session* s, const ox_tensor* logits, ox_tensor** out) {
    OX_TRY
    auto* t = new ox_tensor();
    try {
        t->t = s->s->argmax_last(logits->t);
    } catch (...) {
        delete t;
        throw;
    }
    *out = t;
    return OX_OK;
    OX_CATCH
}

ox_status ox_session_sample_last(ox_session* s, const ox_tensor* logits, float temperature, int64_t top_k, float top_p,
                                 const float* uniform, size_t n_uniform, ox_tensor** out) {
    OX_TRY
    auto* t = new ox_tensor();
    try {
        t->t = s->s->sample_last(logits->t, temperature, (long long)top_k, top_p, uniform, n_uniform);
    } catch (...) {
        delete t;
        throw;
    }
    *out = t;
    return OX_OK;
    OX_CATCH
}

ox_status ox_session_argmax_last_into(ox_session* s, const ox_tensor* logits, ox_tensor* out) {
    OX_TRY
    s->s->argmax_last_into(logits->t, out->t);
    return OX_OK;
    OX_CATCH
}

#ifdef OX_TRACE
// Developer builds only: copy the kernels' trace log (count, then entries) to the host and clear it.
int32_t ox_debug_trace(ox_session* s, uint64_t* out, int32_t cap) {
    s->s->wait_idle();
    char* base = (char*)s->s->error_area() + 256;
    cudaMemcpy(out, base, sizeof(uint64_t) * (size_t)cap, cudaMemcpyDeviceToHost);
    cudaMemset(base, 0, 8);
    return (int32_t)(out[0] & 0xffffffffu);
}
#endif

}  // extern "C"
