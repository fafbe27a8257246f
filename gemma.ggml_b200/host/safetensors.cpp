// safetensors.cpp — see safetensors.h
#include "safetensors.h"

#include <cstdio>
#include <cstring>

#include "json_min.h"

static size_t st_dtype_size(const std::string &d) {
    if (d == "BF16" || d == "F16" || d == "I16" || d == "U16") return 2;
    if (d == "F32" || d == "I32" || d == "U32") return 4;
    if (d == "F64" || d == "I64" || d == "U64") return 8;
    if (d == "I8" || d == "U8" || d == "BOOL") return 1;
    return 0;
}

int safetensors_file::open(const std::string &path, std::string *err) {
    auto fail = [&](const std::string &m) {
        if (err) *err = path + ": " + m;
        return -1;
    };
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) return fail("cannot open");
    fseek(f, 0, SEEK_END);
    const long size = ftell(f);
    fseek(f, 0, SEEK_SET);
    if (size < 8) {
        fclose(f);
        return fail("shorter than a header");
    }
    bytes_.resize((size_t)size);
    const size_t got = fread(bytes_.data(), 1, (size_t)size, f);
    fclose(f);
    if (got != (size_t)size) return fail("short read");
    uint64_t hlen = 0;
    for (int i = 7; i >= 0; i--) hlen = (hlen << 8) | bytes_[(size_t)i];
    if (hlen > (uint64_t)size - 8) return fail("header length beyond the file");
    json_value h;
    std::string jerr;
    if (!json_parser((const char *)bytes_.data() + 8, (size_t)hlen).parse(&h, &jerr)) return fail("header: " + jerr);
    if (h.kind != json_value::OBJ) return fail("header is not an object");
    const uint8_t *data = bytes_.data() + 8 + hlen;
    const size_t data_size = (size_t)size - 8 - (size_t)hlen;
    for (const auto &kv : h.obj) {
        if (kv.first == "__metadata__") continue;
        const json_value &e = kv.second;
        st_tensor t;
        t.dtype = e.string("dtype", "");
        const json_value *sh = e.get("shape"), *off = e.get("data_offsets");
        if (!sh || sh->kind != json_value::ARR || !off || off->kind != json_value::ARR || off->arr.size() != 2)
            return fail("tensor " + kv.first + ": malformed entry");
        for (const auto &d : sh->arr) t.shape.push_back((int64_t)d.num);
        const uint64_t a = (uint64_t)off->arr[0].num, b = (uint64_t)off->arr[1].num;
        const size_t es = st_dtype_size(t.dtype);
        if (!es || b < a || b > data_size || (b - a) != (uint64_t)t.numel() * es)
            return fail("tensor " + kv.first + ": offsets do not fit its shape and type");
        t.data = data + a;
        t.nbytes = (size_t)(b - a);
        tensors_[kv.first] = t;
    }
    return 0;
}
