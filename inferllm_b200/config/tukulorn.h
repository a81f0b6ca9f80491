// Typed configuration of the Tukulorn decoder, read from its config.json keys.
//
// A Tukulorn model lists its layers one by one: `layers[i]` has `type` ("attention": differential attention with two
// score maps per head, biases and a query temperature; "latent_attention": attention through a normed key/value latent
// with rotated channels beside it, a sliding window and a gate per head), `mixer` (the mixer's sizes and constants) and
// `mlp` ({"kind": "dense", "ff": n}, {"kind": "moe", "expert": {"ff": n, "limit": L}, "router": {"experts": E, "top": k,
// "scale": s, "groups": {"count": c, "keep": g}}}, or null for a layer without a feed-forward).  Beside the list: `width`,
// `vocab`, `norm.eps`, optionally `loop` {start, stop, times} (layers start .. stop - 1 run `times` times in a row with
// the same weights and a cache entry per pass; before every pass but the first the embedding output is added to the
// stream) and `max_positions` (the longest sequence; 131072 if not given).  Every layer is a pre-norm block whose
// sublayer outputs pass a learned factor per channel (layer scale) on their way into the stream; norm weights are stored
// around zero.  The output matrix is a tensor of its own.  What the mixers are is said where they are mapped to parts
// (config/tukulorn.cpp).
#pragma once
#include "config/config.h"

namespace illm {

struct TukulornConfig : ArchConfig {
    Json raw;                    // the config.json object as it was read (to_json gives it back)
    long long width = 0, vocab = 0, max_positions = 131072;
    double norm_eps = 1e-6;
    bool has_loop = false;
    long long loop_start = 0, loop_stop = 0, loop_times = 1;

    static std::unique_ptr<ArchConfig> from_json(const Json& d);
    std::string architecture() const override { return "Tukulorn"; }
    Json to_json() const override { return raw; }
    ModelSpec model_spec() const override;
};

}  // namespace illm
