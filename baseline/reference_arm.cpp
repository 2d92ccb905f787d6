// Timing driver for `bench.py --impl reference`: runs the reference project's own, unmodified decoder
// (ai::LocalModel from its include/ai/LocalModel.hpp, CPU kernels, its stub GPU backend) on a model folder
// and prints one JSON object with the seconds it spent.  Nothing of this repository's engine is on this
// path; nothing of the reference is copied here: the headers are included from a checkout.
//
//   reference_arm <model-dir> <ids-file> <n_seqs> <prompt_len> <warmup> <steps> <context> <prefill_seqs> <prefill_len>
//
// <ids-file>: whitespace-separated token ids; the first n_seqs * prompt_len are the decode prompts, the
// next prefill_seqs * prefill_len the prompts of the prefill measurement.
//
// The timed shape is the reference's own (src/LLM.cpp:687-707): one forward over the prompt, then
// `sample -> forward(one token)` per produced token, greedy (temperature 0).  The reference has no batch
// (one cache per conversation, include/ai/LocalModel.hpp:1231-1334), so the sequences run one after
// another and their times add up.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <vector>

#include "ai/LocalModel.hpp"

int main(int argc, char** argv) {
    if (argc < 10) {
        std::fprintf(stderr, "usage: reference_arm <dir> <ids> <n_seqs> <prompt_len> <warmup> <steps> <context> "
                             "<prefill_seqs> <prefill_len>\n");
        return 2;
    }
    const size_t n_seqs = std::strtoull(argv[3], nullptr, 10), prompt_len = std::strtoull(argv[4], nullptr, 10);
    const size_t warmup = std::strtoull(argv[5], nullptr, 10), steps = std::strtoull(argv[6], nullptr, 10);
    const size_t context = std::strtoull(argv[7], nullptr, 10);
    const size_t prefill_seqs = std::strtoull(argv[8], nullptr, 10), prefill_len = std::strtoull(argv[9], nullptr, 10);
    std::vector<size_t> ids;
    {
        std::ifstream in(argv[2]);
        size_t v;
        while (in >> v) ids.push_back(v);
    }
    if (ids.size() < n_seqs * prompt_len + prefill_seqs * prefill_len || prompt_len + warmup + steps > context) {
        std::fprintf(stderr, "reference_arm: too few ids, or the context is too short for the steps\n");
        return 2;
    }
    ai::LocalModel model;
    if (!model.load(argv[1])) { std::fprintf(stderr, "load failed: %s\n", model.error.c_str()); return 1; }
    using clock = std::chrono::steady_clock;
    const auto seconds = [](clock::time_point a, clock::time_point b) { return std::chrono::duration<double>(b - a).count(); };
    math::random::Random rng{0};
    std::vector<float> logits(model.cfg.vocab);

    double decode_s = 0.0, prompt_s = 0.0;
    size_t produced = 0, last_token = 0;
    for (size_t s = 0; s < n_seqs; ++s) {
        ai::LocalCache cache;
        cache.resize(model.cfg, context);
        const clock::time_point p0 = clock::now();
        model.forward(ids.data() + s * prompt_len, prompt_len, cache.length, cache, logits.data());
        prompt_s += seconds(p0, clock::now());
        for (size_t i = 0; i < warmup + steps; ++i) {
            const clock::time_point t0 = clock::now();
            const size_t next = ai::LocalModel::sampleTopK(logits.data(), model.cfg.vocab, 0.0f, 1, rng);
            model.forward(&next, 1, cache.length, cache, logits.data());
            if (i >= warmup) { decode_s += seconds(t0, clock::now()); ++produced; }
            last_token = next;
        }
    }
    double prefill_s = 0.0;
    const size_t base = n_seqs * prompt_len;
    for (size_t s = 0; s < prefill_seqs; ++s) {
        ai::LocalCache cache;
        cache.resize(model.cfg, prefill_len);
        const clock::time_point t0 = clock::now();
        model.forward(ids.data() + base + s * prefill_len, prefill_len, 0, cache, logits.data());
        prefill_s += seconds(t0, clock::now());
    }
    std::printf("{\"decode_seconds\": %.6f, \"decode_tokens\": %zu, \"prompt_seconds\": %.6f, \"prompt_tokens\": %zu, "
                "\"prefill_seconds\": %.6f, \"prefill_tokens\": %zu, \"threads\": %zu, \"last_token\": %zu}\n",
                decode_s, produced, prompt_s, n_seqs * prompt_len, prefill_s, prefill_seqs * prefill_len,
                (size_t)ai::kernels::Pool::instance().size(), last_token);
    return 0;
}
