// The KV-cache generation loop as one native call per step ≙ `LlmSession::step`
// (crates/onyxia-cli/src/llm.rs:110-183) with `discover_kv_pairs` (:232-246):
// present.N.* outputs are fed back as past_key_values.N.* inputs, the cache starts
// empty, masks and other auxiliary inputs are all ones. Greedy sampling runs on the
// device, so a decode step moves 8 + 8·T bytes up and 8 bytes down.
#include <cstring>

#include "../ir/module_api.hpp"
#include "capi_types.hpp"

using namespace ox;

struct ox_llm {
    oxrt::Session* s = nullptr;
    int64_t max_seq_len = 0, past = 0;
    std::vector<std::string> names;             // module inputs, signature order
    std::vector<int> present_of;                // per input: index of the output fed back into it, or −1
    std::vector<oxrt::DTensor> cache;           // per input: the tensor to feed (KV inputs)
    int logits_out = -1;
    std::vector<int64_t> ones;
    int64_t* pinned_tokens = nullptr;           // generate(): where the device drops the tokens
    size_t pinned_cap = 0;
    ~ox_llm() {
        if (pinned_tokens) cudaFreeHost(pinned_tokens);
    }
};

namespace {

std::vector<int64_t> input_shape(const Module& m, size_t i, const Bindings& b) {
    std::vector<int64_t> shp;
    for (auto& d : m.values[m.inputs[i].second].ty.shape) shp.push_back((int64_t)d.eval(b));
    return shp;
}

}  // namespace

#define OX_TRY try {
#define OX_CATCH                                                                          \
    }                                                                                     \
    catch (const ox::Error& e) { return (ox_status)ox::set_error(e); }                    \
    catch (const std::exception& e) { return (ox_status)ox::set_error(ErrKind::Runtime, e.what()); }

extern "C" {

ox_status ox_llm_create(ox_session* session, int64_t max_seq_len, ox_llm** out) {
    OX_TRY
    auto l = std::make_unique<ox_llm>();
    l->s = session->s.get();
    l->max_seq_len = max_seq_len;
    const Module& m = l->s->module();
    const auto& outs = l->s->output_names();
    for (auto& in : m.inputs) l->names.push_back(in.first);
    l->present_of.assign(l->names.size(), -1);
    l->cache.resize(l->names.size());
    for (size_t o = 0; o < outs.size(); o++) {
        if (outs[o] == "logits") l->logits_out = (int)o;
        if (outs[o].rfind("present.", 0) != 0) continue;
        const std::string past = "past_key_values." + outs[o].substr(8);
        for (size_t i = 0; i < l->names.size(); i++)
            if (l->names[i] == past) l->present_of[i] = (int)o;
    }
    if (l->logits_out < 0) fail(ErrKind::Binding, "output 'logits' missing");
    *out = l.release();
    return OX_OK;
    OX_CATCH
}

void ox_llm_free(ox_llm* l) { delete l; }
int64_t ox_llm_sequence_length(const ox_llm* l) { return l->past; }
int32_t ox_llm_logits_dtype(const ox_llm* l) {
    const Module& m = l->s->module();
    return (int32_t)m.values[m.outputs[(size_t)l->logits_out].second].ty.dtype;
}
void ox_llm_reset(ox_llm* l) {
    l->past = 0;
    for (auto& t : l->cache) t = oxrt::DTensor{};
}

// One forward pass over `n_ids` new tokens. With `token_out` the argmax of the last position's logits is
// taken on the device and returned; with `logits_out` the last position's logits are copied out in their
// stored dtype (`logits_cap` bytes available, `logits_written` set).
namespace {
struct SamplingArgs {
    float temperature, top_p, uniform;
    int64_t top_k;
};
ox_status llm_step(ox_llm* l, const int64_t* ids, int32_t n_ids, int64_t* token_out, void* logits_out, size_t logits_cap,
                   size_t* logits_written, const SamplingArgs* sampling, const oxrt::DTensor* ids_dev = nullptr,
                   oxrt::DTensor* token_dev = nullptr);
}  // namespace

ox_status ox_llm_step(ox_llm* l, const int64_t* ids, int32_t n_ids, int64_t* token_out, void* logits_out, size_t logits_cap,
                      size_t* logits_written) {
    return llm_step(l, ids, n_ids, token_out, logits_out, logits_cap, logits_written, nullptr);
}

// The same step with the next token drawn on the device by temperature / top-k / top-p sampling
// (crates/onyxia-cli/src/sampling.rs:36-65) from the caller's uniform number in [0, 1].
ox_status ox_llm_step_sampled(ox_llm* l, const int64_t* ids, int32_t n_ids, float temperature, int64_t top_k, float top_p, float uniform,
                              int64_t* token_out) {
    const SamplingArgs a{temperature, top_p, uniform, top_k};
    return llm_step(l, ids, n_ids, token_out, nullptr, 0, nullptr, &a);
}

// `n_new` greedy tokens in one call: the first step runs `ids` (a prompt, or one token), every later step takes
// its input id from the previous step's argmax without leaving the device. Per step the host still uploads the
// step's attention mask and the device still sends the step's token to (pinned) host memory, but nothing waits for
// the host in between: the steps are enqueued back to back and the call returns when the last token has arrived.
// Generation does not stop at an end-of-sequence id (the caller truncates).
ox_status ox_llm_generate(ox_llm* l, const int64_t* ids, int32_t n_ids, int32_t n_new, int64_t* tokens_out) {
    OX_TRY
    if (n_new <= 0) return OX_OK;
    if (l->past + n_ids + n_new - 1 > l->max_seq_len)
        fail(ErrKind::Shape, "Sequence length " + std::to_string(l->past + n_ids + n_new - 1) + " would exceed max_seq_len " + std::to_string(l->max_seq_len));
    if (l->pinned_cap < (size_t)n_new) {
        if (l->pinned_tokens) cudaFreeHost(l->pinned_tokens);
        l->pinned_tokens = nullptr;
        l->pinned_cap = 0;
        if (cudaMallocHost((void**)&l->pinned_tokens, sizeof(int64_t) * (size_t)n_new) != cudaSuccess) fail(ErrKind::Runtime, "cannot pin host memory for the tokens");
        l->pinned_cap = (size_t)n_new;
    }
    oxrt::DTensor tok;
    for (int32_t i = 0; i < n_new; i++) {
        oxrt::DTensor next;
        const ox_status st = i == 0 ? llm_step(l, ids, n_ids, nullptr, nullptr, 0, nullptr, nullptr, nullptr, &next)
                                    : llm_step(l, nullptr, 1, nullptr, nullptr, 0, nullptr, nullptr, &tok, &next);
        if (st != OX_OK) return st;
        tok = next;
        l->s->download_async(tok, l->pinned_tokens + i);
    }
    l->s->wait_idle();
    std::memcpy(tokens_out, l->pinned_tokens, sizeof(int64_t) * (size_t)n_new);
    return OX_OK;
    OX_CATCH
}

namespace {
ox_status llm_step(ox_llm* l, const int64_t* ids, int32_t n_ids, int64_t* token_out, void* logits_out, size_t logits_cap,
                   size_t* logits_written, const SamplingArgs* sampling, const oxrt::DTensor* ids_dev, oxrt::DTensor* token_dev) {
    OX_TRY
    if (n_ids <= 0) fail(ErrKind::Shape, "Cannot step with empty input_ids");
    if (l->past + n_ids > l->max_seq_len)
        fail(ErrKind::Shape, "Sequence length " + std::to_string(l->past + n_ids) + " would exceed max_seq_len " + std::to_string(l->max_seq_len));
    oxrt::Session& s = *l->s;
    const Module& m = s.module();
    Bindings b;
    auto bind = [&](const char* name, uint64_t v) {
        if (auto id = m.symbols.get(name)) b.bind(*id, v);
    };
    bind("batch_size", 1);
    bind("sequence_length", (uint64_t)n_ids);
    bind("past_sequence_length", (uint64_t)l->past);
    bind("total_sequence_length", (uint64_t)(l->past + n_ids));

    std::vector<std::pair<std::string, oxrt::DTensor>> feed;
    feed.reserve(l->names.size());
    for (size_t i = 0; i < l->names.size(); i++) {
        const std::string& name = l->names[i];
        const DType dt = m.values[m.inputs[i].second].ty.dtype;
        oxrt::DTensor t;
        if (name == "input_ids") {
            if (ids_dev) t = *ids_dev;  // the previous step's token, still on the device
            else t = s.upload(DType::I64, {1, (int64_t)n_ids}, ids, sizeof(int64_t) * (size_t)n_ids);
        } else if (name == "position_ids") {
            std::vector<int64_t> pos((size_t)n_ids);
            for (int j = 0; j < n_ids; j++) pos[j] = l->past + j;
            t = s.upload(DType::I64, {1, (int64_t)n_ids}, pos.data(), sizeof(int64_t) * pos.size());
        } else if (l->present_of[i] >= 0 && l->cache[i].buf) {
            t = l->cache[i];
        } else {
            const std::vector<int64_t> shp = input_shape(m, i, b);
            size_t n = 1;
            for (auto d : shp) n *= (size_t)d;
            const size_t bytes = dtype_storage_bytes(dt, n);
            if (l->present_of[i] >= 0) {  // empty cache on the first step
                std::vector<uint8_t> zeros(bytes, 0);
                t = s.upload(dt, shp, zeros.data(), bytes);
            } else if (dt == DType::I64) {  // masks and friends are all ones (llm.rs:136-151)
                if (l->ones.size() < n) l->ones.assign(std::max<size_t>(n, 4096), 1);
                t = s.upload(dt, shp, l->ones.data(), bytes);
            } else {
                fail(ErrKind::DType, "input '" + name + "' has a dtype the generation loop cannot fill");
            }
        }
        feed.emplace_back(name, std::move(t));
    }
    auto outs = s.run(feed);
    for (size_t i = 0; i < l->names.size(); i++)
        if (l->present_of[i] >= 0) l->cache[i] = outs[(size_t)l->present_of[i]].second;
    l->past += n_ids;
    const oxrt::DTensor& logits = outs[(size_t)l->logits_out].second;
    oxrt::DTensor tok;
    if (token_out && sampling) {
        // the last position's row of a [1, S, V] tensor
        const int64_t vocab = logits.shape.back(), rows = logits.numel() / vocab;
        oxrt::DTensor last = logits;
        last.shape = {1, vocab};
        last.offset += (size_t)(rows - 1) * dtype_storage_bytes(logits.dtype, (uint64_t)vocab);
        tok = s.sample_last(last, sampling->temperature, (long long)sampling->top_k, sampling->top_p, &sampling->uniform, 1);
    } else if (token_out || token_dev) {
        tok = s.argmax_last(logits);
    }
    if (token_dev) {  // the last position's id as a [1, 1] tensor: the next step's input_ids
        *token_dev = tok;
        const int64_t n = tok.numel();
        token_dev->offset += (size_t)(n - 1) * sizeof(int64_t);
        token_dev->shape = {1, 1};
    }
    // While the device works on this step, get the plan of the next one-token step ready.
    if (l->past + 1 <= l->max_seq_len) {
        std::vector<std::pair<std::string, oxrt::DTensor>> next;
        next.reserve(l->names.size());
        bool ok = true;
        for (size_t i = 0; i < l->names.size() && ok; i++) {
            oxrt::DTensor t;
            if (l->present_of[i] >= 0) {
                t = l->cache[i];
            } else {
                t.dtype = m.values[m.inputs[i].second].ty.dtype;
                if (l->names[i] == "input_ids" || l->names[i] == "position_ids") t.shape = {1, 1};
                else if (l->names[i] == "attention_mask") t.shape = {1, l->past + 1};
                else ok = false;  // an auxiliary input this loop cannot predict
            }
            next.emplace_back(l->names[i], std::move(t));
        }
        if (ok) s.preplan(next);
    }
    if (token_out) {
        std::vector<int64_t> host((size_t)std::max<int64_t>(tok.numel(), 1));
        size_t written = 0;
        s.download(tok, host.data(), host.size() * sizeof(int64_t), &written);
        *token_out = host[(size_t)tok.numel() - 1];
    }
    if (logits_out) {
        // the last position's row
        const int64_t vocab = logits.shape.back(), rows = logits.numel() / vocab;
        const size_t row_bytes = dtype_storage_bytes(logits.dtype, (uint64_t)vocab);
        if (logits_cap < row_bytes) fail(ErrKind::Shape, "logits buffer too small");
        oxrt::DTensor last = logits;
        last.shape = {vocab};
        last.offset += (size_t)(rows - 1) * row_bytes;
        s.download(last, logits_out, logits_cap, logits_written);
    }
    return OX_OK;
    OX_CATCH
}
}  // namespace

}  // extern "C"
