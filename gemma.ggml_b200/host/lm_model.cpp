// lm_model.cpp — the architecture registry (see lm_model.h)
#include "lm_model.h"

#include <cstdio>
#include <map>

static std::map<std::string, lm_factory> &registry() {
    static std::map<std::string, lm_factory> r;
    return r;
}

void lm_register(const char *architecture, lm_factory f) { registry()[architecture] = f; }

std::vector<std::string> lm_architectures() {
    std::vector<std::string> v;
    for (const auto &kv : registry()) v.push_back(kv.first);
    return v;
}

lm_model *lm_load(const std::string &dir, const lm_load_options &opt, std::string *err) {
    const std::string path = dir + "/config.json";
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) {
        if (err) *err = path + ": cannot open";
        return nullptr;
    }
    std::string text;
    char buf[4096];
    size_t n;
    while ((n = fread(buf, 1, sizeof buf, f)) > 0) text.append(buf, n);
    fclose(f);
    return lm_load_config(text, dir, opt, err);
}

lm_model *lm_load_config(const std::string &text, const std::string &dir, const lm_load_options &opt, std::string *err) {
    const std::string path = dir.empty() ? "configuration" : dir + "/config.json";
    json_value cfg;
    std::string jerr;
    if (!json_parser(text.data(), text.size()).parse(&cfg, &jerr) || cfg.kind != json_value::OBJ) {
        if (err) *err = path + ": " + (jerr.empty() ? "not an object" : jerr);
        return nullptr;
    }
    const std::string arch = cfg.string("architecture", "");
    auto it = registry().find(arch);
    if (it == registry().end()) {
        if (err) {
            *err = path + ": architecture '" + arch + "' is not registered (known:";
            for (const auto &a : lm_architectures()) *err += " " + a;
            *err += ")";
        }
        return nullptr;
    }
    return it->second(dir, cfg, opt, err);
}
