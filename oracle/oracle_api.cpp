// TEST INFRASTRUCTURE — C entry points of the CPU oracle, for the test-suite,
// the smoke check and the benchmark's CPU-baseline leg (ctypes).
// ≙ onyxia_backend_ref::{RefBackend, RefSession, run_once}
// (crates/onyxia-backend-ref/src/lib.rs:46-107).
#include <cstring>

#include "../onyxia_b200/csrc/ir/module_api.hpp"
#include "interp.hpp"

using namespace ox;

struct oxref_session {
    oxref::RefSession s;
};

struct oxref_result {
    std::vector<std::pair<std::string, oxref::Tensor>> outs;
};

#define OX_TRY try {
#define OX_CATCH                                                     \
    }                                                                \
    catch (const ox::Error& e) { return ox::set_error(e); }          \
    catch (const std::exception& e) { return ox::set_error(ErrKind::Runtime, e.what()); }

extern "C" {

void oxref_set_threads(int n) { oxref::set_threads(n); }
void oxref_set_allreduce_hook(oxref::AllReduceHook hook) { oxref::allreduce_hook() = hook; }
int oxref_get_threads(void) { return oxref::get_threads(); }

// Inline every composite and validate; consumes the module.
int oxref_prepare(ox_module* m, oxref_session** out) {
    OX_TRY
    std::unique_ptr<ox_module> owned(m);
    auto* s = new oxref_session();
    try {
        s->s = oxref::prepare(std::move(owned->b.module()));
    } catch (...) {
        delete s;
        throw;
    }
    *out = s;
    return 0;
    OX_CATCH
}

void oxref_session_free(oxref_session* s) { delete s; }
int oxref_session_num_nodes(const oxref_session* s) { return (int)s->s.module.nodes.size(); }

// Run on host tensors. Input bytes are borrowed for the duration of the call.
int oxref_run(const oxref_session* s, const char* const* names, const int32_t* dtypes, const uint64_t* const* shapes,
              const int32_t* ranks, const void* const* datas, const size_t* nbytes, int32_t n_in, oxref_result** out) {
    OX_TRY
    std::vector<std::pair<std::string, oxref::Tensor>> ins;
    for (int i = 0; i < n_in; i++) {
        std::vector<size_t> shape(shapes[i], shapes[i] + ranks[i]);
        oxref::Tensor t = oxref::Tensor::view((DType)dtypes[i], shape, (const uint8_t*)datas[i]);
        if (t.nbytes() != nbytes[i])
            fail(ErrKind::Interp, "tensor data size mismatch for input '" + std::string(names[i]) + "'");
        ins.emplace_back(names[i], std::move(t));
    }
    auto* r = new oxref_result();
    try {
        r->outs = s->s.run(ins);
    } catch (...) {
        delete r;
        throw;
    }
    *out = r;
    return 0;
    OX_CATCH
}

int oxref_result_count(const oxref_result* r) { return (int)r->outs.size(); }
const char* oxref_result_name(const oxref_result* r, int i) { return r->outs[i].first.c_str(); }
int oxref_result_dtype(const oxref_result* r, int i) { return (int)r->outs[i].second.dtype; }
int oxref_result_rank(const oxref_result* r, int i) { return (int)r->outs[i].second.shape.size(); }
void oxref_result_shape(const oxref_result* r, int i, uint64_t* out) {
    auto& s = r->outs[i].second.shape;
    for (size_t d = 0; d < s.size(); d++) out[d] = s[d];
}
const void* oxref_result_data(const oxref_result* r, int i) { return r->outs[i].second.data; }
size_t oxref_result_nbytes(const oxref_result* r, int i) { return r->outs[i].second.nbytes(); }
void oxref_result_free(oxref_result* r) { delete r; }

// Conversions the tests use to pin the f16 rounding.
uint16_t oxref_f64_to_f16(double v) { return f64_to_f16_bits(v); }
double oxref_f16_to_f64(uint16_t h) { return f16_bits_to_f64(h); }

}  // extern "C"
