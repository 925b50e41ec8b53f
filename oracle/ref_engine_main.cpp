// TEST INFRASTRUCTURE ONLY.  Drives the reference's own engine (qw3::Engine, include/qw3/qw3.hpp) on a GGUF file
// with a token-id prompt (GenerationOptions::prompt_token_ids_override, include/qw3/qw3.hpp:232-237) and prints the
// generated text on stdout; the engine's own log lines (native mtp_spec_summary: / mtp_accept_hist:,
// src/qwen_native_backend.cpp:16313-16392) go to stderr untouched.  Linked from the reference's host sources and its
// CUDA DeviceBackend where they lie (oracle/Makefile target ref-engine); nothing here is part of the product.
//
//   qw3ref_engine <model.gguf> <greedy|mtp> <chain k> <max_tokens> <ctx> <token id> [<token id> ...]
//
// Sampling requests (GenerationOptions temperature / top_p / top_k / min_p / seed / presence_penalty / repetition_penalty,
// include/qw3/qw3.hpp:224-230) come from the environment: QW3REF_TEMPERATURE (default 0 = greedy), QW3REF_TOP_P,
// QW3REF_TOP_K, QW3REF_MIN_P, QW3REF_SEED, QW3REF_PRESENCE, QW3REF_REPETITION.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <exception>
#include <string>
#include <vector>

#include "qw3/qw3.hpp"

int main(int argc, char **argv) {
    if (argc < 7) {
        std::fprintf(stderr, "usage: %s model.gguf greedy|mtp k max_tokens ctx token...\n", argv[0]);
        return 2;
    }
    try {
        qw3::EngineOptions eo;
        eo.model_path = argv[1];
        eo.backend = qw3::BackendKind::QwenNative;
        const bool mtp = std::strcmp(argv[2], "mtp") == 0;
        eo.native_mtp_speculate = mtp;
        eo.native_mtp_chain = std::atoi(argv[3]);
        eo.native_mtp_chain_set = mtp;
        eo.native_linear_backend = "custom";
        eo.ctx_size = std::atoi(argv[5]);
        eo.verbose = true;
        qw3::GenerationOptions go;
        go.max_tokens = std::atoi(argv[4]);
        auto envf = [](const char *name, double dflt) { const char *v = std::getenv(name); return v && *v ? std::atof(v) : dflt; };
        go.temperature = (float)envf("QW3REF_TEMPERATURE", 0.0);
        go.top_k = (int)envf("QW3REF_TOP_K", 0.0);
        go.top_p = (float)envf("QW3REF_TOP_P", 1.0);
        go.min_p = (float)envf("QW3REF_MIN_P", 0.0);
        go.presence_penalty = (float)envf("QW3REF_PRESENCE", 0.0);
        go.repetition_penalty = (float)envf("QW3REF_REPETITION", 1.0);
        if (const char *v = std::getenv("QW3REF_SEED")) go.seed = std::strtoull(v, nullptr, 10);
        go.raw_prompt = true;
        go.ignore_eos = true;
        for (int i = 6; i < argc; ++i) go.prompt_token_ids_override.push_back((uint32_t)std::strtoul(argv[i], nullptr, 10));
        qw3::Engine engine(eo);
        const std::string text = engine.generate("", go);
        std::printf("QW3REF_TEXT %s\n", text.c_str());
        return 0;
    } catch (const std::exception &e) {
        std::fprintf(stderr, "qw3ref_engine: %s\n", e.what());
        return 1;
    }
}
