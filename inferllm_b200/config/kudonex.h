// Typed configuration of the Kudonex decoder, read from its config.json keys.
//
// A Kudonex model lists its layers one by one: `layers[i]` has `type` ("mlstm", "mamba2" or "attention": which
// mixer), `mixer` (the mixer's sizes and constants) and `mlp` ({"kind": "moe", "expert": {"ff": n}, "router":
// {"experts": E, "top": k, "groups": {"count": c, "keep": g}}, "shared": {"ff": n}}, or null for a layer without a
// feed-forward).  Beside the list: `width`, `vocab`, `norm.eps`, `embedding.scale`, optionally `canon.taps` (every
// mixer then reads its input plus a short causal convolution of it) and `max_positions` (the longest sequence;
// 131072 if not given).  Every layer norms each sublayer's input and output (layer norms with a weight and no bias);
// a sinusoid position vector is added to the scaled token embedding; the output matrix is the embedding table.  What
// the three mixers are is said where they are mapped to parts (config/kudonex.cpp).
#pragma once
#include "config/config.h"

namespace illm {

struct KudonexConfig : ArchConfig {
    Json raw;                    // the config.json object as it was read (to_json gives it back)
    long long width = 0, vocab = 0, max_positions = 131072;
    double norm_eps = 1e-5, embedding_scale = 1.0;
    long long canon_taps = 0;    // 0: no input convolution

    static std::unique_ptr<ArchConfig> from_json(const Json& d);
    std::string architecture() const override { return "Kudonex"; }
    Json to_json() const override { return raw; }
    ModelSpec model_spec() const override;
};

}  // namespace illm
