// Test driver for edge_fm::CompactVocab (host logic only, no GPU): loads an engine JSON, applies one
// operation to the ids on the command line and prints "ok <ids...>" or "error <Type> <message>".
//   compact_vocab_check <engine.json> info|remap|required|restore|embed <ints...>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "compact_vocab.h"

using namespace edge_fm;

int main(int argc, char** argv) {
    if (argc < 3) return 2;
    const std::string op = argv[2];
    std::vector<int32_t> ids;
    for (int i = 3; i < argc; ++i) ids.push_back((int32_t)std::atoi(argv[i]));
    try {
        EngineConfig cfg(argv[1]);
        CompactVocab cv(cfg);
        std::vector<int32_t> out;
        if (op == "info") out = {cv.enabled() ? 1 : 0, cv.original_vocab_size(), cv.compact_vocab_size()};
        else if (op == "remap") out = cv.remap_token_ids(ids, "request token_ids");
        else if (op == "required") out = cv.remap_required_token_ids(ids, "sampling.stop_token_ids");
        else if (op == "restore") out = cv.restore_token_ids(ids, "response token_ids");
        else if (op == "embed") out = {cv.remap_embed_token_id(ids.at(0), ids.at(1))};
        else return 2;
        std::printf("ok");
        for (int32_t v : out) std::printf(" %d", v);
        std::printf("\n");
    } catch (const InvalidRequestError& e) {
        std::printf("error InvalidRequestError %s\n", e.what());
    } catch (const ConfigurationError& e) {
        std::printf("error ConfigurationError %s\n", e.what());
    } catch (const InternalError& e) {
        std::printf("error InternalError %s\n", e.what());
    } catch (const std::exception& e) {
        std::printf("error other %s\n", e.what());
    }
    return 0;
}
