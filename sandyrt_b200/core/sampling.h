// Sampling options of a request, with the reference's names and meanings, and the uniform
// numbers behind sampled tokens.
//
// src/server/Sampler.h:13-22 of the reference: SamplingConfig{topK = 1, topP = 1.0,
// temperature = 0.0}, per-request overrides of temperature and top_p; checked by
// resolveSamplingConfig (src/server/Sampler.cpp:111-125): top_k > 0, 0 < top_p <= 1,
// temperature >= 0 and finite.  temperature 0 is greedy.  One difference: the reference's default
// top_k = 1 makes every draw greedy until a model's model_config.json raises it
// (src/server/Model.cpp:63-96).  Here top_k = 0 means "no top-k cut" and is the default, so
// `temperature` alone switches sampling on.
//
// Drawing itself runs on the device (csrc/sampling.cu, launched by the step function).  The
// uniform number behind every draw comes from a counter-based generator keyed by the request's
// seed and the index of the token being drawn, so a request's tokens do not depend on which other
// requests share its steps.  (The reference draws on the host from one std::mt19937_64 per
// sampler, src/server/Sampler.cpp:127-131, serving one request at a time.)
#pragma once

#include <cmath>
#include <cstdint>
#include <optional>

#include "errors.h"

namespace sandy {

struct SamplingParams {
    float temperature = 0.0f;
    int top_k = 0;                       // 0: whole vocabulary
    float top_p = 1.0f;
    std::optional<uint64_t> seed;        // nullopt: a fresh seed per request

    void validate() const {
        if (top_k < 0) throw ValueError("top_k must be >= 0 (0 keeps the whole vocabulary)");
        if (!std::isfinite(top_p) || top_p <= 0.0f || top_p > 1.0f) throw ValueError("top_p must be > 0 and <= 1");
        if (!std::isfinite(temperature) || temperature < 0.0f) throw ValueError("temperature must be >= 0");
    }
    bool greedy() const { return temperature == 0.0f || top_k == 1; }
};

inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    uint64_t z = x;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// The uniform number in [0, 1) for token `index` of a request with `seed` (24 bits, so it is
// exact in float32).
inline float uniform_for(uint64_t seed, uint64_t index) {
    const uint64_t h = splitmix64(splitmix64(seed) + index);
    return (float)(h >> 40) / 16777216.0f;
}

uint64_t fresh_seed();       // from the system's entropy source

}  // namespace sandy
