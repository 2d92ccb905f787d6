// Driver for tests/golden/make_golden.py: runs the reference's ai::LocalModel on
// a model folder and writes float32 logits of every position, twice: from calls
// that feed the prompt up to and including each position in one forward, and
// from feeding one token at a time into one cache.
//
//   local_model_probe <model-dir> <out.bin> <id> <id> ...
//
// Compiled against the reference's headers; nothing of the reference is copied.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "ai/LocalModel.hpp"

int main(int argc, char** argv) {
    if (argc < 4) { std::fprintf(stderr, "usage: probe <dir> <out> ids...\n"); return 2; }
    std::vector<size_t> ids;
    for (int i = 3; i < argc; ++i) ids.push_back(std::strtoull(argv[i], nullptr, 10));

    ai::LocalModel model;
    if (!model.load(argv[1])) { std::fprintf(stderr, "load failed: %s\n", model.error.c_str()); return 1; }
    const size_t vocab = model.cfg.vocab, n = ids.size();
    std::vector<float> whole(n * vocab), stepwise(n * vocab);

    // forward() returns the last row only, so the logits of position t come from a prefill of t+1 tokens
    for (size_t t = 0; t < n; ++t) {
        ai::LocalCache cache;
        cache.resize(model.cfg, n);
        model.forward(ids.data(), t + 1, 0, cache, whole.data() + t * vocab);
    }
    {
        ai::LocalCache cache;
        cache.resize(model.cfg, n);
        for (size_t t = 0; t < n; ++t)
            model.forward(&ids[t], 1, cache.length, cache, stepwise.data() + t * vocab);
    }
    std::FILE* f = std::fopen(argv[2], "wb");
    if (!f) return 1;
    std::fwrite(whole.data(), sizeof(float), whole.size(), f);
    std::fwrite(stepwise.data(), sizeof(float), stepwise.size(), f);
    std::fclose(f);
    return 0;
}
