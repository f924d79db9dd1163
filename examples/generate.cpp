// Generate tokens from a model folder with the engine's C++ API; no Python in the process.
//
//   make -C examples                      (builds the host library, the kernel libraries and this program)
//   examples/generate MODEL_DIR [--dtype bfloat16|float32] [--max-tokens 16] [--temperature 0] [--seed 0] 1 2 3 ...
//
// MODEL_DIR holds config.json and model.safetensors (write one with seeded random weights:
// `python -m sandyrt_b200 random-model --config configs/gpt2_small.json --out DIR`).  The trailing
// numbers are the prompt's token ids.  Prints the generated ids and the finish reason.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "sandy/llm.h"

int main(int argc, char** argv) {
    if (argc < 3) {
        std::fprintf(stderr, "usage: %s MODEL_DIR [--dtype bfloat16|float32] [--max-tokens N] [--temperature T] [--seed S] ID...\n", argv[0]);
        return 2;
    }
    sandy::LLMOptions options;
    sandy::GenerateParams params;
    std::vector<int> prompt;
    for (int i = 2; i < argc; i++) {
        const std::string a = argv[i];
        if (a == "--dtype" && i + 1 < argc) options.dtype = std::strcmp(argv[++i], "float32") == 0 ? sandy::DType::F32 : sandy::DType::BF16;
        else if (a == "--max-tokens" && i + 1 < argc) params.max_tokens = std::atoi(argv[++i]);
        else if (a == "--temperature" && i + 1 < argc) params.temperature = (float)std::atof(argv[++i]);
        else if (a == "--seed" && i + 1 < argc) params.seed = (uint64_t)std::atoll(argv[++i]);
        else prompt.push_back(std::atoi(a.c_str()));
    }
    options.cache_tokens = 4096;
    options.max_live = 4;
    try {
        std::unique_ptr<sandy::LLM> llm = sandy::LLM::load(argv[1], options);
        params.on_token = [](int, int token) { std::printf("%d ", token); std::fflush(stdout); return true; };
        const std::vector<sandy::GenerateResult> results = llm->generate({prompt}, params);
        std::printf("\nfinish_reason=%s prompt_tokens=%d completion_tokens=%d decode_toks_per_s=%.1f\n",
                    results[0].finish_reason.c_str(), results[0].prompt_tokens, results[0].completion_tokens,
                    results[0].decode_tokens_per_second);
    } catch (const sandy::Error& e) {
        std::fprintf(stderr, "%s: %s\n", e.kind().c_str(), e.what());
        return 1;
    }
    return 0;
}
