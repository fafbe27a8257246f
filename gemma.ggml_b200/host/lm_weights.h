// lm_weights.h — where a model's numbers come from: the tensors of a .safetensors file (bf16 or fp32, any byte
// offset), or a counter-based generator for throughput runs and tests of other sizes.  Header-only.
#pragma once

#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "safetensors.h"

static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static inline uint16_t f32_to_bf16(float f) { // round to nearest even
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static inline int tensor_f32(const st_tensor &t, std::vector<float> *out) {
    const size_t n = (size_t)t.numel();
    out->resize(n);
    if (t.dtype == "BF16") {
        for (size_t i = 0; i < n; i++) {
            uint16_t h;
            memcpy(&h, t.data + 2 * i, 2);
            (*out)[i] = bf16_to_f32(h);
        }
    } else if (t.dtype == "F32") {
        memcpy(out->data(), t.data, n * 4);
    } else {
        return -1;
    }
    return 0;
}

// where a layer's numbers come from: the file, or a counter-based generator for throughput runs
struct weight_source {
    const safetensors_file *file;
    uint64_t seed;
    std::string *err;
    uint64_t counter = 0;
    static uint64_t mix(uint64_t x) {
        x += 0x9E3779B97F4A7C15ull;
        x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
        x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
        return x ^ (x >> 31);
    }
    // rows x cols numbers of `name`; random: uniform in +-amp around `mean`
    int get(const std::string &name, int64_t rows, int64_t cols, float amp, float mean, std::vector<float> *out) {
        if (file) {
            const st_tensor *t = file->find(name);
            if (!t) {
                *err = "tensor '" + name + "' is missing";
                return -1;
            }
            if (t->numel() != rows * cols) {
                *err = "tensor '" + name + "' has " + std::to_string(t->numel()) + " numbers, the configuration asks for " +
                       std::to_string(rows) + " x " + std::to_string(cols);
                return -1;
            }
            if (tensor_f32(*t, out)) {
                *err = "tensor '" + name + "': type " + t->dtype + " is not read";
                return -1;
            }
            return 0;
        }
        const uint64_t key = mix(seed + 0xD1B54A32D192ED03ull * ++counter);
        out->resize((size_t)(rows * cols));
        for (size_t i = 0; i < out->size(); i++) {
            const uint64_t r = mix(key + i);
            (*out)[i] = mean + amp * (float)((double)(r >> 11) / 9007199254740992.0 * 2.0 - 1.0);
        }
        return 0;
    }
    // 1 when the tensor holds one number (file), as `dflt` says otherwise
    int numel(const std::string &name, int dflt) const {
        if (!file) return dflt;
        const st_tensor *t = file->find(name);
        return t ? (int)t->numel() : -1;
    }
};

