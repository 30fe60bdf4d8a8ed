// Compact-vocabulary translation on the generate() boundary ("edgefm.compact_vocab.v1").
// Same contract and public interface as the reference's CompactVocab
// (src/engine/tasks/token_generation/compact_vocab.{h,cpp}, doc/compact_vocab_contract.md): callers keep
// speaking original tokenizer ids; the checkpoint is pre-pruned to compact_vocab_size rows, request ids /
// stop ids / prefix ids are translated old -> new before the model runs and generated ids new -> old
// before they reach Response.token_ids().  A pruned id is an error, never a silent fallback.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "config.h"
#include "edge-fm/core.h"

namespace edge_fm {

class CompactVocab {
public:
    CompactVocab() = default;                               // disabled: every call is the identity
    explicit CompactVocab(const EngineConfig& config);      // reads compact_vocab.{enabled,mapping_path,reject_unknown_input_ids}

    bool enabled() const noexcept { return enabled_; }
    int32_t original_vocab_size() const noexcept { return (int32_t)old_to_new_.size(); }
    int32_t compact_vocab_size() const noexcept { return (int32_t)new_to_old_.size(); }
    const std::string& mapping_path() const noexcept { return mapping_path_; }

    // ids that arrive with a request: an absent id is the caller's fault (InvalidRequestError)
    std::vector<int32_t> remap_token_ids(const std::vector<int32_t>& ids, const std::string& context) const;
    // ids the deployment depends on (EOS, configured stop ids, special ids, KV prefixes): absent = ConfigurationError
    std::vector<int32_t> remap_required_token_ids(const std::vector<int32_t>& ids, const std::string& context) const;
    std::vector<int32_t> remap_optional_token_ids(const std::vector<int32_t>& ids, const std::string& context) const;
    // generated compact ids back to tokenizer ids; out of range = InternalError
    std::vector<int32_t> restore_token_ids(const std::vector<int32_t>& ids, const std::string& context) const;

    // First compact id of a request's custom-embedding placeholders [embed_token_id, embed_token_id + n): every
    // placeholder must be kept and the range must stay contiguous.  Negative ids pass through.
    int32_t remap_embed_token_id(int32_t embed_token_id, int64_t num_custom_embeddings) const;

private:
    enum class Blame { Request, Deployment };
    int32_t forward(int32_t id, const std::string& context, Blame blame) const;

    bool enabled_ = false;
    std::string mapping_path_;
    std::vector<int32_t> old_to_new_;     // -1: pruned
    std::vector<int32_t> new_to_old_;
};

}  // namespace edge_fm
