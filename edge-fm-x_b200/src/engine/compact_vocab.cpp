#include "compact_vocab.h"

#include <fstream>
#include <sstream>

namespace edge_fm {

namespace {

const char kFormat[] = "edgefm.compact_vocab.v1";

[[noreturn]] void bad_mapping(const std::string& why) { throw ConfigurationError("compact_vocab mapping: " + why); }

int32_t int_field(const json::Value& m, const char* key) {
    const json::Value* v = m.find(key);
    if (v == nullptr || !v->is_number() || !v->is_int) bad_mapping(std::string("integer field required: ") + key);
    return (int32_t)v->inum;
}

std::vector<int32_t> int_list(const json::Value& m, const char* key) {
    const json::Value* v = m.find(key);
    if (v == nullptr || !v->is_array()) bad_mapping(std::string("integer array field required: ") + key);
    std::vector<int32_t> out;
    out.reserve(v->arr.size());
    for (const json::Value& e : v->arr) {
        if (!e.is_number() || !e.is_int) bad_mapping(std::string("field ") + key + " must contain only integers");
        out.push_back((int32_t)e.inum);
    }
    return out;
}

std::string describe(const std::string& context, int32_t id) { return context + " token id " + std::to_string(id); }

}  // namespace

CompactVocab::CompactVocab(const EngineConfig& config) {
    const json::Value opts = config.compact_vocab();
    if (!opts.get_bool("enabled", false)) return;
    if (!opts.get_bool("reject_unknown_input_ids", true))
        throw ConfigurationError("compact_vocab v1 requires reject_unknown_input_ids=true: no remap is defined for unknown tokens");
    const std::string raw = opts.get_string("mapping_path", "");
    if (raw.empty()) throw ConfigurationError("compact_vocab.enabled=true requires compact_vocab.mapping_path");
    mapping_path_ = raw[0] == '/' ? raw : config.config_dir() + "/" + raw;      // relative to the engine JSON

    std::ifstream f(mapping_path_);
    if (!f.is_open()) throw ConfigurationError("Cannot open compact_vocab mapping file: " + mapping_path_);
    std::ostringstream text;
    text << f.rdbuf();
    json::Value m;
    try {
        m = json::parse(text.str());
    } catch (const std::exception& e) {
        throw ConfigurationError("Failed to parse compact_vocab mapping file " + mapping_path_ + ": " + e.what());
    }
    if (m.get_string("format", "") != kFormat) bad_mapping(std::string("format must be ") + kFormat);
    const int32_t n_old = int_field(m, "original_vocab_size"), n_new = int_field(m, "compact_vocab_size");
    if (n_old <= 0 || n_new <= 0) bad_mapping("vocabulary sizes must be positive");
    if (n_new > n_old) bad_mapping("compact_vocab_size must be <= original_vocab_size");
    old_to_new_ = int_list(m, "old_to_new");
    new_to_old_ = int_list(m, "new_to_old");
    if ((int32_t)old_to_new_.size() != n_old) bad_mapping("old_to_new length must equal original_vocab_size");
    if ((int32_t)new_to_old_.size() != n_new) bad_mapping("new_to_old length must equal compact_vocab_size");
    // ranges first, then: the two tables must be exact inverses on the kept ids
    for (int32_t c = 0; c < n_new; ++c)
        if (new_to_old_[c] < 0 || new_to_old_[c] >= n_old)
            bad_mapping("new_to_old holds an out-of-range original id at compact id " + std::to_string(c));
    for (int32_t o = 0; o < n_old; ++o)
        if (old_to_new_[o] < -1 || old_to_new_[o] >= n_new)
            bad_mapping("old_to_new holds an out-of-range compact id at original id " + std::to_string(o));
    for (int32_t c = 0; c < n_new; ++c)
        if (old_to_new_[new_to_old_[c]] != c) bad_mapping("new_to_old / old_to_new disagree at compact id " + std::to_string(c));
    for (int32_t o = 0; o < n_old; ++o)
        if (old_to_new_[o] >= 0 && new_to_old_[old_to_new_[o]] != o)
            bad_mapping("old_to_new / new_to_old disagree at original id " + std::to_string(o));
    // the checkpoint must already be pruned
    const json::Value mc = config.prefill_model_config();
    const json::Value* vs = mc.find("vocab_size");
    if (vs == nullptr || !vs->is_number()) throw ConfigurationError("compact_vocab requires config.json to define integer vocab_size");
    if ((int32_t)vs->inum != n_new)
        throw ConfigurationError("compact_vocab v1 expects a pre-pruned checkpoint: config.json vocab_size=" + std::to_string(vs->inum) +
                                 ", compact_vocab_size=" + std::to_string(n_new));
    enabled_ = true;
    // everything the deployment relies on must have survived the pruning
    (void)remap_required_token_ids(int_list(m, "special_token_ids"), "compact_vocab.special_token_ids");
    (void)remap_required_token_ids(config.eos_token_ids(), "model eos_token_ids");
    (void)remap_required_token_ids(config.stop_token_ids(), "sampling.stop_token_ids");
}

int32_t CompactVocab::forward(int32_t id, const std::string& context, Blame blame) const {
    if (!enabled_) return id;
    const bool kept = id >= 0 && id < (int32_t)old_to_new_.size() && old_to_new_[id] >= 0;
    if (kept) return old_to_new_[id];
    if (blame == Blame::Request)
        throw InvalidRequestError("compact_vocab cannot remap " + describe(context, id) + "; the token is absent from old_to_new");
    throw ConfigurationError("compact_vocab requires " + describe(context, id) + " to be present in old_to_new");
}

std::vector<int32_t> CompactVocab::remap_token_ids(const std::vector<int32_t>& ids, const std::string& context) const {
    std::vector<int32_t> out(ids);
    if (enabled_)
        for (int32_t& id : out) id = forward(id, context, Blame::Request);
    return out;
}

std::vector<int32_t> CompactVocab::remap_required_token_ids(const std::vector<int32_t>& ids, const std::string& context) const {
    std::vector<int32_t> out(ids);
    if (enabled_)
        for (int32_t& id : out) id = forward(id, context, Blame::Deployment);
    return out;
}

std::vector<int32_t> CompactVocab::remap_optional_token_ids(const std::vector<int32_t>& ids, const std::string& context) const {
    return remap_required_token_ids(ids, context);
}

std::vector<int32_t> CompactVocab::restore_token_ids(const std::vector<int32_t>& ids, const std::string& context) const {
    std::vector<int32_t> out(ids);
    if (!enabled_) return out;
    for (int32_t& id : out) {
        if (id < 0 || id >= (int32_t)new_to_old_.size())
            throw InternalError("compact_vocab cannot restore " + describe(context, id) + "; compact id is out of range");
        id = new_to_old_[id];
    }
    return out;
}

int32_t CompactVocab::remap_embed_token_id(int32_t embed_token_id, int64_t num_custom_embeddings) const {
    if (!enabled_ || embed_token_id < 0) return embed_token_id;
    if (num_custom_embeddings < 0) throw InvalidRequestError("compact_vocab requires embeddings to expose their row count in shape[0]");
    const int32_t first = forward(embed_token_id, "request embed_token_id", Blame::Request);
    for (int64_t i = 1; i < num_custom_embeddings; ++i) {
        const int32_t c = forward(embed_token_id + (int32_t)i, "request embedding placeholder", Blame::Request);
        if (c != first + (int32_t)i)
            throw InvalidRequestError("compact_vocab requires custom embedding placeholder ids to remap to a contiguous range. old_base=" +
                                      std::to_string(embed_token_id) + ", compact_base=" + std::to_string(first) + ", offset=" +
                                      std::to_string(i) + ", compact_id=" + std::to_string(c));
    }
    return first;
}

}  // namespace edge_fm
