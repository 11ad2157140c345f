// Run-time reader for kleos_config.json and the sizes derived from it.
//
// The reference turns the same JSON file into -D macros at CMake time
// (csrc/CMakeLists.txt:184-252) and derives every size in the compile-time struct ACC
// (csrc/include/kleos/types.cuh:442-513).  Here the file is parsed when the layer is
// initialised.  Keys and enum values follow csrc/kleos_config.schema.json:5-89; the one
// extension is that capacity_factor may be fractional.
#pragma once

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>

namespace kleos {

struct LayerConfig {
    double capacity_factor = 1;
    int drop_tokens = 1, expert_top_k = 2, global_batch = 0, is_training = 0, hidden_act = 0;
    int hidden_size = 0, intermediate_size = 0, mini_batch = 1, moe_frequency = 1;
    int num_experts = 0, num_layers = 1, sequence_len = 0, torch_dtype = 0, vocab_size = 0;

    // derived (types.cuh:471-508)
    int S = 0, H = 0, I = 0, E = 0, K = 0, PX = 0, EC = 0, pEC = 0, elem_bytes = 0;

    static int ceil_div(long long a, long long b) { return static_cast<int>((a + b - 1) / b); }

    // Returns an empty string on success, otherwise what is wrong.
    std::string derive() {
        if (torch_dtype < 0 || torch_dtype > 3) return "torch_dtype must be 0..3";
        if (hidden_act != 0 && hidden_act != 1) return "hidden_act must be 0 (relu) or 1 (gelu)";
        if (hidden_size <= 0 || hidden_size % 64) return "hidden_size must be a positive multiple of 64";
        if (intermediate_size <= 0 || intermediate_size % 64)
            return "intermediate_size must be a positive multiple of 64";
        if (sequence_len <= 0 || sequence_len % 128) return "sequence_len must be a positive multiple of 128";
        if (mini_batch < 1) return "mini_batch must be >= 1";
        if (num_experts < 1 || num_experts > 65535) return "num_experts must be in [1, 65535]";
        if (expert_top_k < 1 || expert_top_k > num_experts) return "expert_top_k must be in [1, num_experts]";
        if (capacity_factor < 1) return "capacity_factor must be >= 1";
        S = sequence_len * mini_batch;
        H = hidden_size;
        I = intermediate_size;
        E = num_experts;
        K = expert_top_k;
        PX = ceil_div(E, 64) * 64;
        const long long base = drop_tokens ? ceil_div(S, E) : S;
        EC = static_cast<int>(std::ceil(base * capacity_factor - 1e-9)) * K;
        pEC = ceil_div(EC, 128) * 128;
        elem_bytes = (torch_dtype == 0 || torch_dtype == 1) ? 4 : 2;
        return "";
    }
};

// Minimal parser for a flat JSON object whose values are numbers (the whole schema).
inline std::string parse_flat_json(const std::string& text, std::map<std::string, double>* out) {
    size_t i = 0;
    const size_t n = text.size();
    auto skip_ws = [&]() {
        while (i < n && (text[i] == ' ' || text[i] == '\n' || text[i] == '\t' || text[i] == '\r')) ++i;
    };
    skip_ws();
    if (i >= n || text[i] != '{') return "expected '{'";
    ++i;
    for (;;) {
        skip_ws();
        if (i < n && text[i] == '}') return "";
        if (i >= n || text[i] != '"') return "expected a quoted key";
        const size_t k0 = ++i;
        while (i < n && text[i] != '"') ++i;
        if (i >= n) return "unterminated key";
        const std::string key = text.substr(k0, i - k0);
        ++i;
        skip_ws();
        if (i >= n || text[i] != ':') return "expected ':' after key " + key;
        ++i;
        skip_ws();
        if (text.compare(i, 4, "true") == 0) {
            (*out)[key] = 1;
            i += 4;
        } else if (text.compare(i, 5, "false") == 0) {
            (*out)[key] = 0;
            i += 5;
        } else {
            char* end = nullptr;
            const double v = std::strtod(text.c_str() + i, &end);
            if (end == text.c_str() + i) return "value of " + key + " is not a number";
            (*out)[key] = v;
            i = static_cast<size_t>(end - text.c_str());
        }
        skip_ws();
        if (i < n && text[i] == ',') {
            ++i;
            continue;
        }
        if (i < n && text[i] == '}') return "";
        return "expected ',' or '}' after " + key;
    }
}

inline std::string load_config(const char* path, LayerConfig* cfg) {
    FILE* f = std::fopen(path, "rb");
    if (!f) return std::string("cannot open ") + path;
    std::string text;
    char buf[4096];
    size_t got;
    while ((got = std::fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, got);
    std::fclose(f);
    std::map<std::string, double> kv;
    std::string err = parse_flat_json(text, &kv);
    if (!err.empty()) return err;
    // required keys: kleos_config.schema.json:74-89
    static const char* required[] = {"capacity_factor", "drop_tokens", "expert_top_k", "is_training",
                                     "hidden_act", "hidden_size", "intermediate_size", "mini_batch",
                                     "moe_frequency", "num_experts", "num_layers", "sequence_len",
                                     "torch_dtype", "vocab_size"};
    for (const char* k : required)
        if (!kv.count(k)) return std::string("missing required key ") + k;
    auto geti = [&](const char* k, int dflt) { return kv.count(k) ? static_cast<int>(kv[k]) : dflt; };
    cfg->capacity_factor = kv["capacity_factor"];
    cfg->drop_tokens = geti("drop_tokens", 1);
    cfg->expert_top_k = geti("expert_top_k", 2);
    cfg->global_batch = geti("global_batch", 0);
    cfg->is_training = geti("is_training", 0);
    cfg->hidden_act = geti("hidden_act", 0);
    cfg->hidden_size = geti("hidden_size", 0);
    cfg->intermediate_size = geti("intermediate_size", 0);
    cfg->mini_batch = geti("mini_batch", 1);
    cfg->moe_frequency = geti("moe_frequency", 1);
    cfg->num_experts = geti("num_experts", 0);
    cfg->num_layers = geti("num_layers", 1);
    cfg->sequence_len = geti("sequence_len", 0);
    cfg->torch_dtype = geti("torch_dtype", 0);
    cfg->vocab_size = geti("vocab_size", 0);
    return cfg->derive();
}

}  // namespace kleos
